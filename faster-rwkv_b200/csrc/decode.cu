// Persistent whole-token decode kernel for sm_100a.
//
// One cooperative launch runs a whole token (all layers + head) for up to 8 independent streams.
// grid = one CTA per SM.  Each CTA has one producer warp and NW consumer warps:
//   * the producer walks the CTA's static list of weight tiles (a function of phase index and CTA id
//     only) and keeps a ring of shared-memory stages full with 1-D TMA bulk copies; weights do not
//     depend on activations, so it runs ahead across phase boundaries and HBM stays busy while the
//     consumers sit in a grid barrier;
//   * the consumers stage the phase's input vectors in shared memory as fp16 tensor-core operands
//     (LayerNorm + token-shift mix fused here), then for every 16-row block multiply the streamed
//     tile with mma.sync.m16n8k16 (weights = A operand, streams = B operand columns, fp32
//     accumulation, int8/int4 dequantised in registers), reduce across the warps that split K, and
//     apply the phase's epilogue (WKV state update + sigmoid gate, residual add, squared ReLU, ...).
//     Each activation is fed as two fp16 columns, hi = fp16(x) and lo = fp16(x - hi), whose results
//     are added: the operand keeps ~22 mantissa bits at no extra MMA for one stream (7 of the 8
//     columns are idle anyway) and 4 streams share one MMA.
// Phases are separated by a grid barrier (release/acquire counter in global memory).  Every wait
// is bounded: after WAIT_LIMIT_NS it records a status and the CTA drains without hanging.
#include "common.cuh"
#include "internal.h"

namespace frb {

namespace {

constexpr int BAR_CONS = 1;  // named barrier id of the consumer warps

struct Smem {
  uint64_t *full, *empty;
  volatile int *abort_flag;
  float *ln_red;     // [NW][2*MAX_B]
  float *stats;      // [2*MAX_B] mean, rstd
  float *stash;      // [MAX_B][STASH_N] LayerNorm outputs of the channels whose shift state this CTA writes
  float *red;        // [2][3][NW][RED_N]
  __half *xs;        // operand vectors
  uint8_t *ring;
};
constexpr int STASH_N = 128;

// NB = operand columns kept per n-tile (2: one stream as hi/lo; 8: four streams as hi/lo), NT = n-tiles.
template <int NB, int NT> __host__ __device__ constexpr int n_streams() { return NB == 2 ? 1 : 4 * NT; }
template <int NB, int NT> __host__ __device__ constexpr int red_n() { return ROWS * n_streams<NB, NT>(); }

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <int NB, int NT>
__host__ __device__ inline size_t smem_layout(size_t xs_halfs, int n_stages, size_t *off_stash, size_t *off_red,
                                              size_t *off_xs, size_t *off_ring) {
  size_t o = 1024;  // barriers + flags + LN scratch
  *off_stash = o; o += sizeof(float) * n_streams<NB, NT>() * STASH_N;
  *off_red = o;   o += sizeof(float) * 2 * 3 * NW * red_n<NB, NT>();
  o = align_up(o, 128);
  *off_xs = o;    o += xs_halfs * 2;
  o = align_up(o, 1024);
  *off_ring = o;  o += (size_t)n_stages * SLOT_BYTES;
  return o;
}

__host__ __device__ inline size_t xs_halfs_needed(int C, int F, int version, int NB, int NT) {
  size_t a = (size_t)(version == 4 ? 3 : 4) * C;
  size_t b = F;
  return (a > b ? a : b) * NB * NT;
}

// ------------------------------------------------------------------------------------------------
// stage x operand -> accumulators.  acc[e][t]: two interleaved accumulator sets e (breaks the MMA
// dependency chain), n-tile t.
template <int FMT, int NB, int NT>
__device__ __forceinline__ void process_stage(const uint8_t *st, int nch, const __half *xv, size_t plane_u4, int chunk0,
                                              int warp, int lane, float acc[2][NT][4]) {
  const int g = lane >> 2, q = lane & 3;
  const int n = NB == 2 ? (g & 1) : g;   // operand column this lane feeds
  const uint4 *xb = reinterpret_cast<const uint4 *>(xv);
  for (int c = warp; c < nch; c += NW) {
    const size_t xo = ((size_t)(chunk0 + c) * 2 * NB + n) * 4 + q;
    uint4 b01[NT], b23[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      b01[t] = xb[xo + t * plane_u4];            // MMAs 0,1 of the chunk
      b23[t] = xb[xo + t * plane_u4 + NB * 4];   // MMAs 2,3
    }
    if (FMT == FMT_FP16) {
      const uint4 *A = reinterpret_cast<const uint4 *>(st + (size_t)c * 2048) + lane;
      const uint4 a0 = A[0], a1 = A[32], a2 = A[64], a3 = A[96];
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        mma16816(acc[0][t], a0.x, a0.y, a0.z, a0.w, b01[t].x, b01[t].y);
        mma16816(acc[1][t], a1.x, a1.y, a1.z, a1.w, b01[t].z, b01[t].w);
        mma16816(acc[0][t], a2.x, a2.y, a2.z, a2.w, b23[t].x, b23[t].y);
        mma16816(acc[1][t], a3.x, a3.y, a3.z, a3.w, b23[t].z, b23[t].w);
      }
    } else if (FMT == FMT_INT8) {
      const uint4 *A = reinterpret_cast<const uint4 *>(st + (size_t)c * 1024) + lane;
      const uint4 w01 = A[0], w23 = A[32];
      const uint32_t M = 0x64646464u, OFF = 0x64806480u;  // 1024 + byte, minus 1152 -> byte - 128
#define FRB_I8(w, sel) hsub2_u32(prmt(w, M, sel), OFF)
      {
        const uint32_t p0 = FRB_I8(w01.x, 0x4140), p1 = FRB_I8(w01.x, 0x4342), p2 = FRB_I8(w01.y, 0x4140),
                       p3 = FRB_I8(w01.y, 0x4342);
        const uint32_t r0 = FRB_I8(w01.z, 0x4140), r1 = FRB_I8(w01.z, 0x4342), r2 = FRB_I8(w01.w, 0x4140),
                       r3 = FRB_I8(w01.w, 0x4342);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma16816(acc[0][t], p0, p1, p2, p3, b01[t].x, b01[t].y);
          mma16816(acc[1][t], r0, r1, r2, r3, b01[t].z, b01[t].w);
        }
      }
      {
        const uint32_t p0 = FRB_I8(w23.x, 0x4140), p1 = FRB_I8(w23.x, 0x4342), p2 = FRB_I8(w23.y, 0x4140),
                       p3 = FRB_I8(w23.y, 0x4342);
        const uint32_t r0 = FRB_I8(w23.z, 0x4140), r1 = FRB_I8(w23.z, 0x4342), r2 = FRB_I8(w23.w, 0x4140),
                       r3 = FRB_I8(w23.w, 0x4342);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma16816(acc[0][t], p0, p1, p2, p3, b23[t].x, b23[t].y);
          mma16816(acc[1][t], r0, r1, r2, r3, b23[t].z, b23[t].w);
        }
      }
#undef FRB_I8
    } else {
      const uint4 w = (reinterpret_cast<const uint4 *>(st + (size_t)c * 512))[lane];
      const uint2 scw = *reinterpret_cast<const uint2 *>(st + (size_t)nch * 512 + (size_t)c * 64 + g * 8);
      const float2 s0 = __half22float2(*reinterpret_cast<const __half2 *>(&scw.x));  // group 0: rows g, g+8
      const float2 s1 = __half22float2(*reinterpret_cast<const __half2 *>(&scw.y));  // group 1
      const uint32_t LO = 0x000f000fu, HI = 0x00f000f0u, M0 = 0x64006400u, M1 = 0x54005400u;
      const uint32_t O0 = 0x64086408u, O1 = 0x54805480u;  // 1024+8, 64+8
#define FRB_I4(wd, t0, t1, t2, t3)                                   \
  const uint32_t t0 = hsub2_u32(lop3_and_or(wd, LO, M0), O0);        \
  const uint32_t t1 = hsub2_u32(lop3_and_or(wd, HI, M1), O1);        \
  const uint32_t t2 = hsub2_u32(lop3_and_or((wd) >> 8, LO, M0), O0); \
  const uint32_t t3 = hsub2_u32(lop3_and_or((wd) >> 8, HI, M1), O1);
      {
        FRB_I4(w.x, p0, p1, p2, p3)
        FRB_I4(w.y, r0, r1, r2, r3)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          float s[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816(s, p0, p1, p2, p3, b01[t].x, b01[t].y);
          mma16816(s, r0, r1, r2, r3, b01[t].z, b01[t].w);
          acc[0][t][0] += s0.x * s[0]; acc[0][t][1] += s0.x * s[1];
          acc[0][t][2] += s0.y * s[2]; acc[0][t][3] += s0.y * s[3];
        }
      }
      {
        FRB_I4(w.z, p0, p1, p2, p3)
        FRB_I4(w.w, r0, r1, r2, r3)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          float s[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816(s, p0, p1, p2, p3, b23[t].x, b23[t].y);
          mma16816(s, r0, r1, r2, r3, b23[t].z, b23[t].w);
          acc[1][t][0] += s1.x * s[0]; acc[1][t][1] += s1.x * s[1];
          acc[1][t][2] += s1.y * s[2]; acc[1][t][3] += s1.y * s[3];
        }
      }
#undef FRB_I4
    }
  }
}

// ------------------------------------------------------------------------------------------------
struct Ctx {
  const DecodeParams *p;
  Smem sm;
  int tid, warp, lane, cta, G;
  int slot;            // ring position of the next stage
  uint32_t parity;     // parity of the next full-barrier wait
  unsigned epoch;      // grid barriers passed
  int own0, ownn;      // channels whose shift state this CTA writes
  uint8_t *stash_dst;  // pending shift-state write (per-stream base + b*state_stride), or null
};

__device__ __forceinline__ int token_id(const DecodeParams &p, int b) {
  return p.ids_dev ? __ldcg(p.ids_dev + b) : p.ids_val[b];
}

__device__ __forceinline__ void grid_barrier(Ctx &cx) {
  const DecodeParams &p = *cx.p;
  bar_sync(BAR_CONS, NCONS);
  if (cx.tid == 0) {
    cx.epoch++;
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync) : "memory");
    const unsigned target = cx.epoch * (unsigned)cx.G;
    unsigned v;
    unsigned long long t0 = 0;
    int it = 0;
    while (true) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.sync) : "memory");
      if ((int)(v - target) >= 0) break;
      if (*cx.sm.abort_flag) break;
      if ((++it & 1023) == 0) {
        if (t0 == 0) t0 = globaltimer_ns();
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS || __ldcg(p.status) != 0) {
          *cx.sm.abort_flag = 1;
          atomicCAS(p.status, 0, ST_TIMEOUT_GRID);
          break;
        }
      }
    }
    __threadfence();
  }
  bar_sync(BAR_CONS, NCONS);
}

// write the stashed LayerNorm outputs into the token-shift state (after the barrier that follows
// the phase which read the old state)
__device__ __forceinline__ void flush_stash(Ctx &cx) {
  if (!cx.stash_dst) return;
  const DecodeParams &p = *cx.p;
  const int n = cx.ownn * p.B;
  for (int t = cx.tid; t < n; t += NCONS) {
    const int b = t / cx.ownn, i = t - b * cx.ownn;
    const float v = cx.sm.stash[b * STASH_N + i];
    uint8_t *dst = cx.stash_dst + (size_t)b * p.state_stride;
    if (p.act_fp16) reinterpret_cast<__half *>(dst)[cx.own0 + i] = __float2half_rn(v);
    else reinterpret_cast<float *>(dst)[cx.own0 + i] = v;
  }
  cx.stash_dst = nullptr;
}

__device__ __forceinline__ float4 load_act4(const uint8_t *base, int i4, int act_fp16) {
  if (act_fp16) {
    const uint2 u = __ldcg(reinterpret_cast<const uint2 *>(base) + i4);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  return __ldcg(reinterpret_cast<const float4 *>(base) + i4);
}

// Operand position of stream b inside a vector: n-tile plane and the hi / lo columns.
template <int NB>
__device__ __forceinline__ void operand_cols(int b, int &tile, int &col_hi, int &col_lo) {
  if (NB == 2) { tile = 0; col_hi = 0; col_lo = 1; }
  else { tile = b >> 2; col_hi = b & 3; col_lo = 4 + (b & 3); }
}

// Write 4 consecutive inputs k..k+3 of stream b into operand vector `vec` as hi + lo fp16 columns.
template <int NB>
__device__ __forceinline__ void store_operand4(__half *vec, size_t plane_halfs, int k, int b, float a, float bb, float c,
                                               float dd) {
  int tile, ch, cl;
  operand_cols<NB>(b, tile, ch, cl);
  __half *pl = vec + (size_t)tile * plane_halfs;
  const __half2 h0 = __floats2half2_rn(a, bb), h1 = __floats2half2_rn(c, dd);
  const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
  const __half2 l0 = __floats2half2_rn(a - f0.x, bb - f0.y), l1 = __floats2half2_rn(c - f1.x, dd - f1.y);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t *>(&h0); u.y = *reinterpret_cast<const uint32_t *>(&h1);
  *reinterpret_cast<uint2 *>(pl + xs_index(k, ch, NB)) = u;
  u.x = *reinterpret_cast<const uint32_t *>(&l0); u.y = *reinterpret_cast<const uint32_t *>(&l1);
  *reinterpret_cast<uint2 *>(pl + xs_index(k, cl, NB)) = u;
}

// Residual stream column b, float4 index i4: the embedding row at layer 0, else x.
__device__ __forceinline__ float4 load_x4(const DecodeParams &p, int layer0, int b, int i4) {
  if (layer0) {
    if (p.emb_f32)
      return __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.emb) + (size_t)token_id(p, b) * p.C) + i4);
    const __half *row = reinterpret_cast<const __half *>(p.emb) + (size_t)token_id(p, b) * p.C;
    const uint2 u = __ldg(reinterpret_cast<const uint2 *>(row) + i4);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
    const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
    return make_float4(a.x, a.y, c.x, c.y);
  }
  return __ldcg(reinterpret_cast<const float4 *>(p.x + (size_t)b * p.C) + i4);
}

// LayerNorm statistics of the residual stream for all B columns -> sm.stats (mean[b], rstd[b]).
// Shifted single pass: sums of (x - x[0]) and (x - x[0])^2 in fp32.
template <int SB>
__device__ __forceinline__ void ln_stats(Ctx &cx, int layer0) {
  constexpr int NB = SB;  // one slot per stream
  const DecodeParams &p = *cx.p;
  const int n4 = p.C >> 2;
  float s1[NB], s2[NB], piv[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    s1[b] = s2[b] = 0.f;
    piv[b] = b < p.B ? load_x4(p, layer0, b, 0).x : 0.f;
  }
  for (int i4 = cx.tid; i4 < n4; i4 += NCONS) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      if (b < p.B) {
        const float4 v = load_x4(p, layer0, b, i4);
        const float d0 = v.x - piv[b], d1 = v.y - piv[b], d2 = v.z - piv[b], d3 = v.w - piv[b];
        s1[b] += (d0 + d1) + (d2 + d3);
        s2[b] += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s1[b] += __shfl_xor_sync(0xffffffffu, s1[b], o);
      s2[b] += __shfl_xor_sync(0xffffffffu, s2[b], o);
    }
  }
  if (cx.lane == 0) {
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      cx.sm.ln_red[cx.warp * 2 * MAX_B + 2 * b] = s1[b];
      cx.sm.ln_red[cx.warp * 2 * MAX_B + 2 * b + 1] = s2[b];
    }
  }
  bar_sync(BAR_CONS, NCONS);
  if (cx.tid < NB && cx.tid < p.B) {
    const int b = cx.tid;
    float a = 0.f, c = 0.f;
    for (int w = 0; w < NW; ++w) {
      a += cx.sm.ln_red[w * 2 * MAX_B + 2 * b];
      c += cx.sm.ln_red[w * 2 * MAX_B + 2 * b + 1];
    }
    const float inv = 1.f / (float)p.C;
    const float m = a * inv;
    float var = c * inv - m * m;
    var = var > 0.f ? var : 0.f;
    cx.sm.stats[2 * b] = load_x4(p, layer0, b, 0).x + m;  // same pivot every thread used
    cx.sm.stats[2 * b + 1] = rsqrtf(var + 1e-5f);
  }
  bar_sync(BAR_CONS, NCONS);
}

// LayerNorm + token-shift mix: writes nvec operand vectors (fp16) into sm.xs, stashes LN output of
// the owned channels for the deferred shift-state write.  nvec == 0: plain LayerNorm -> xs[0].
template <int NB, int NT>
__device__ __forceinline__ void prologue_ln_mix(Ctx &cx, int layer0, const float *ln_w, const float *ln_b,
                                                const float *const *mix, int nvec, const uint8_t *sx_state) {
  constexpr int SB = n_streams<NB, NT>();
  const DecodeParams &p = *cx.p;
  ln_stats<SB>(cx, layer0);
  const int n4 = p.C >> 2;
  const size_t plane = (size_t)p.C * NB;   // halfs per (vector, n-tile)
  const size_t vstride = plane * NT;       // halfs per operand vector
  for (int i4 = cx.tid; i4 < n4; i4 += NCONS) {
    const float4 gw = __ldg(reinterpret_cast<const float4 *>(ln_w) + i4);
    const float4 gb = __ldg(reinterpret_cast<const float4 *>(ln_b) + i4);
    float4 mx[4];
#pragma unroll
    for (int v = 0; v < 4; ++v)
      if (v < nvec) mx[v] = __ldg(reinterpret_cast<const float4 *>(mix[v]) + i4);
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      if (b >= p.B) break;
      const float mean = cx.sm.stats[2 * b], rstd = cx.sm.stats[2 * b + 1];
      const float4 xv = load_x4(p, layer0, b, i4);
      float4 xx;
      xx.x = (xv.x - mean) * rstd * gw.x + gb.x;
      xx.y = (xv.y - mean) * rstd * gw.y + gb.y;
      xx.z = (xv.z - mean) * rstd * gw.z + gb.z;
      xx.w = (xv.w - mean) * rstd * gw.w + gb.w;
      if (nvec == 0) {
        store_operand4<NB>(cx.sm.xs, plane, i4 * 4, b, xx.x, xx.y, xx.z, xx.w);
        continue;
      }
      const float4 sx = load_act4(sx_state + (size_t)b * p.state_stride, i4, p.act_fp16);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        if (v < nvec) {
          const float4 m = mx[v];
          store_operand4<NB>(cx.sm.xs + v * vstride, plane, i4 * 4, b, xx.x * m.x + sx.x * (1.f - m.x),
                             xx.y * m.y + sx.y * (1.f - m.y), xx.z * m.z + sx.z * (1.f - m.z),
                             xx.w * m.w + sx.w * (1.f - m.w));
        }
      }
      const int c = i4 * 4 - cx.own0;
      if (c > -4 && c < cx.ownn) {
        float *st = cx.sm.stash + b * STASH_N;
        if (c >= 0 && c < cx.ownn) st[c] = xx.x;
        if (c + 1 >= 0 && c + 1 < cx.ownn) st[c + 1] = xx.y;
        if (c + 2 >= 0 && c + 2 < cx.ownn) st[c + 2] = xx.z;
        if (c + 3 >= 0 && c + 3 < cx.ownn) st[c + 3] = xx.w;
      }
    }
  }
  bar_sync(BAR_CONS, NCONS);
}

// fp32 vector [B][K] in global memory -> operand vector 0
template <int NB, int NT>
__device__ __forceinline__ void prologue_vec(Ctx &cx, const float *src, int K) {
  constexpr int SB = n_streams<NB, NT>();
  const DecodeParams &p = *cx.p;
  const int n4 = K >> 2;
  const size_t plane = (size_t)K * NB;
  for (int i4 = cx.tid; i4 < n4; i4 += NCONS) {
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      if (b >= p.B) break;
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)b * K) + i4);
      store_operand4<NB>(cx.sm.xs, plane, i4 * 4, b, v.x, v.y, v.z, v.w);
    }
  }
  bar_sync(BAR_CONS, NCONS);
}

// v5 output projection input: GroupNorm over each head's 64 readout values, times the gate
template <int NB, int NT>
__device__ __forceinline__ void prologue_gn_gate(Ctx &cx, const LayerDev &ly) {
  constexpr int SB = n_streams<NB, NT>();
  const DecodeParams &p = *cx.p;
  const size_t plane = (size_t)p.C * NB;
  const int n4 = p.C >> 2;  // 16 float4 per head -> 16 consecutive threads share a head
  for (int base = 0; base < n4; base += NCONS) {
    const int i4 = base + cx.tid;
    const bool ok = i4 < n4;
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      if (b >= p.B) break;
      float4 v = ok ? __ldcg(reinterpret_cast<const float4 *>(p.o5 + (size_t)b * p.C) + i4) : make_float4(0, 0, 0, 0);
      float s = (v.x + v.y) + (v.z + v.w);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s * (1.f / 64.f);
      const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
      float q = (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
      const float rstd = rsqrtf(q * (1.f / 64.f) + 1e-5f);
      if (ok) {
        const float4 gw = __ldg(reinterpret_cast<const float4 *>(ly.lnx_w) + i4);
        const float4 gb = __ldg(reinterpret_cast<const float4 *>(ly.lnx_b) + i4);
        float4 y = make_float4(d0 * rstd * gw.x + gb.x, d1 * rstd * gw.y + gb.y, d2 * rstd * gw.z + gb.z,
                               d3 * rstd * gw.w + gb.w);
        if (p.version >= 51) {
          const float4 g = __ldcg(reinterpret_cast<const float4 *>(p.g5 + (size_t)b * p.C) + i4);
          y.x *= g.x; y.y *= g.y; y.z *= g.z; y.w *= g.w;
        }
        store_operand4<NB>(cx.sm.xs, plane, i4 * 4, b, y.x, y.y, y.z, y.w);
      }
    }
  }
  bar_sync(BAR_CONS, NCONS);
}

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// ---- epilogue of one (row, stream) output --------------------------------------------------------
__device__ __forceinline__ void epilogue(const DecodeParams &p, const PhaseDev &ph, const LayerDev *ly, int it,
                                         int row, int b, const float val[3]) {
  const int C = p.C;
  switch (ph.kind) {
    case PH_ATT_KVR: {
      const int c = it * ROWS + row;
      uint8_t *st = p.state + (size_t)b * p.state_stride + (size_t)ph.layer * p.layer_stride;
      float *aa = reinterpret_cast<float *>(st + (size_t)C * act_bytes(p.act_fp16));
      float *bb = aa + C, *pp = bb + C;
      const float k = val[0], v = val[1], r = sigmoid_f(val[2]);
      const float u = __ldg(ly->first + c), w = __ldg(ly->decay + c);
      const float a0 = aa[c], b0 = bb[c], p0 = pp[c];
      float ww = u + k;
      float pm = fmaxf(p0, ww);
      float e1 = expf(p0 - pm), e2 = expf(ww - pm);
      const float wkv = (e1 * a0 + e2 * v) / (e1 * b0 + e2);
      p.rwkv[(size_t)b * C + c] = r * wkv;
      ww = w + p0;
      pm = fmaxf(ww, k);
      e1 = expf(ww - pm);
      e2 = expf(k - pm);
      aa[c] = e1 * a0 + e2 * v;
      bb[c] = e1 * b0 + e2;
      pp[c] = pm;
      break;
    }
    case PH_ATT_O: {
      const int c = it * ROWS + row;
      float xin;
      if (ph.layer == 0)
        xin = p.emb_f32 ? __ldg(reinterpret_cast<const float *>(p.emb) + (size_t)token_id(p, b) * C + c)
                        : __half2float(reinterpret_cast<const __half *>(p.emb)[(size_t)token_id(p, b) * C + c]);
      else xin = __ldcg(p.x + (size_t)b * C + c);
      p.x[(size_t)b * C + c] = xin + val[0];
      break;
    }
    case PH_FFN_KR: {
      if (it < ph.split[0]) {
        const int f = it * ROWS + row;
        const float t = fmaxf(val[0], 0.f);
        p.kk[(size_t)b * p.F + f] = t * t;
      } else {
        const int c = (it - ph.split[0]) * ROWS + row;
        p.rr[(size_t)b * C + c] = sigmoid_f(val[0]);
      }
      break;
    }
    case PH_FFN_V: {
      const int c = it * ROWS + row;
      float xn = __ldcg(p.x + (size_t)b * C + c) + __ldcg(p.rr + (size_t)b * C + c) * val[0];
      if (p.rescale_every > 0 && (ph.layer + 1) % p.rescale_every == 0) xn *= 0.5f;
      p.x[(size_t)b * C + c] = xn;
      break;
    }
    case PH_MATVEC:
    case PH_HEAD: {
      const int v = it * ROWS + row;
      p.logits[(size_t)b * p.Vpad + v] = val[0];
      break;
    }
    case PH5_KVRG: {
      const int nb = C / ROWS;
      const int cls = it / nb, c = (it - cls * nb) * ROWS + row;
      float *dst = cls == 0 ? p.k5 : cls == 1 ? p.v5 : cls == 2 ? p.r5 : p.g5;
      float v = val[0];
      if (cls == 3) v = v * sigmoid_f(v);
      dst[(size_t)b * C + c] = v;
      break;
    }
    default: break;
  }
}

// ---- all row blocks of a phase that belong to this CTA ----------------------------------------------
template <int FMT, int NB, int NT>
__device__ __forceinline__ void run_items(Ctx &cx, const PhaseDev &ph, const LayerDev *ly) {
  constexpr int SB = n_streams<NB, NT>();
  constexpr int RN = red_n<NB, NT>();
  const DecodeParams &p = *cx.p;
  const int KT = kt_max(FMT);
  const int nst = num_stages(FMT, ph.K);
  const size_t plane = (size_t)ph.K * NB;   // halfs per (vector, n-tile)
  const size_t vstride = plane * NT;
  int buf = 0;
  const int first = (cx.cta + cx.G - ph.rot) % cx.G;
  for (int it = first; it < ph.n_items; it += cx.G) {
    float acc[3][2][NT][4];
#pragma unroll
    for (int u = 0; u < 3; ++u)
#pragma unroll
      for (int e = 0; e < 2; ++e)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[u][e][t][i] = 0.f;
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      if (u < ph.n_sub) {
        // which operand vector feeds this matrix
        int vec = u;
        if (ph.kind == PH_FFN_KR) vec = it < ph.split[0] ? 0 : 1;
        else if (ph.kind == PH5_KVRG) vec = it / (p.C / ROWS);
        const __half *xv = cx.sm.xs + (size_t)vec * vstride;
        for (int s = 0; s < nst; ++s) {
          const int kt = min(KT, ph.K - s * KT);
          mbar_wait(&cx.sm.full[cx.slot], cx.parity, cx.sm.abort_flag, p.status, ST_TIMEOUT_FULL);
          process_stage<FMT, NB, NT>(cx.sm.ring + (size_t)cx.slot * SLOT_BYTES, kt / CHUNK_K, xv, plane / 8,
                                     s * (KT / CHUNK_K), cx.warp, cx.lane, acc[u]);
          __syncwarp();
          if (cx.lane == 0) mbar_arrive(&cx.sm.empty[cx.slot]);
          if (++cx.slot == p.n_stages) { cx.slot = 0; cx.parity ^= 1u; }
        }
      }
    }
    // hi + lo columns, then the cross-warp reduction of the K split.  Accumulator c0,c1 = row g,
    // columns 2q, 2q+1; c2,c3 = row g+8.
    float *red = cx.sm.red + (size_t)buf * 3 * NW * RN;
    const int g = cx.lane >> 2, q = cx.lane & 3;
#pragma unroll
    for (int u = 0; u < 3; ++u) {
      if (u < ph.n_sub) {
        float *r = red + ((size_t)u * NW + cx.warp) * RN;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          float c0 = acc[u][0][t][0] + acc[u][1][t][0], c1 = acc[u][0][t][1] + acc[u][1][t][1];
          float c2 = acc[u][0][t][2] + acc[u][1][t][2], c3 = acc[u][0][t][3] + acc[u][1][t][3];
          if (NB == 2) {
            // columns 0 (hi) and 1 (lo) of the q == 0 lanes
            if (q == 0) { r[g] = c0 + c1; r[g + 8] = c2 + c3; }
          } else {
            // columns 0..3 = hi of streams 0..3 (lanes q = 0,1), columns 4..7 = lo (lanes q = 2,3)
            c0 += __shfl_xor_sync(0xffffffffu, c0, 2);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 2);
            c2 += __shfl_xor_sync(0xffffffffu, c2, 2);
            c3 += __shfl_xor_sync(0xffffffffu, c3, 2);
            if (q < 2) {
              const int sb = t * 4 + 2 * q;
              r[g * SB + sb] = c0; r[g * SB + sb + 1] = c1;
              r[(g + 8) * SB + sb] = c2; r[(g + 8) * SB + sb + 1] = c3;
            }
          }
        }
      }
    }
    bar_sync(BAR_CONS, NCONS);
    if (cx.tid < ROWS * SB) {
      const int row = cx.tid / SB, b = cx.tid % SB;
      if (b < p.B) {
        float val[3] = {0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < 3; ++u) {
          if (u < ph.n_sub) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) s += red[((size_t)u * NW + w) * RN + cx.tid];
            if (FMT == FMT_INT8) s *= __half2float(__ldg(ph.rscale + ((size_t)it * ph.n_sub + u) * ROWS + row));
            val[u] = s;
          }
        }
        epilogue(p, ph, ly, it, row, b, val);
      }
    }
    buf ^= 1;
  }
}

// ---- v5 state update + readout: units of (stream, head, 16 value columns) ----------------------------
__device__ __forceinline__ void phase_wkv5(Ctx &cx, const PhaseDev &ph, const LayerDev &ly) {
  const DecodeParams &p = *cx.p;
  const int C = p.C, H = p.H;
  const int units = p.B * H * 4;
  float *scratch = reinterpret_cast<float *>(cx.sm.xs);  // [NW][16] partial readouts
  const int first = (cx.cta + cx.G - ph.rot) % cx.G;
  for (int un = first; un < units; un += cx.G) {
    const int b = un / (H * 4), h = (un / 4) % H, j0 = (un & 3) * 16;
    const int i = cx.tid >> 2, jq = (cx.tid & 3) * 4;
    uint8_t *stb = p.state + (size_t)b * p.state_stride + (size_t)ph.layer * p.layer_stride;
    float *S = reinterpret_cast<float *>(stb + (size_t)C * act_bytes(p.act_fp16)) + (size_t)h * 4096;
    float4 *sp = reinterpret_cast<float4 *>(S + i * 64 + j0 + jq);
    float4 s = *sp;
    const float ki = __ldcg(p.k5 + (size_t)b * C + h * 64 + i), ri = __ldcg(p.r5 + (size_t)b * C + h * 64 + i);
    const float4 vj = __ldcg(reinterpret_cast<const float4 *>(p.v5 + (size_t)b * C + h * 64 + j0 + jq));
    const float u = p.version == 50 ? __ldg(ly.first + h) : __ldg(ly.first + h * 64 + i);
    const float w = p.version == 50 ? __ldg(ly.decay + h) : __ldg(ly.decay + h * 64 + i);
    const float a0 = ki * vj.x, a1 = ki * vj.y, a2 = ki * vj.z, a3 = ki * vj.w;
    float o0 = ri * (u * a0 + s.x), o1 = ri * (u * a1 + s.y), o2 = ri * (u * a2 + s.z), o3 = ri * (u * a3 + s.w);
    s.x = a0 + w * s.x; s.y = a1 + w * s.y; s.z = a2 + w * s.z; s.w = a3 + w * s.w;
    *sp = s;
    // sum over the 8 key rows held by this warp (lanes with equal lane & 3)
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      o0 += __shfl_xor_sync(0xffffffffu, o0, o);
      o1 += __shfl_xor_sync(0xffffffffu, o1, o);
      o2 += __shfl_xor_sync(0xffffffffu, o2, o);
      o3 += __shfl_xor_sync(0xffffffffu, o3, o);
    }
    if (cx.lane < 4) {
      float *d = scratch + cx.warp * 16 + cx.lane * 4;
      d[0] = o0; d[1] = o1; d[2] = o2; d[3] = o3;
    }
    bar_sync(BAR_CONS, NCONS);
    if (cx.tid < 16) {
      float t = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < NW; ++w8) t += scratch[w8 * 16 + cx.tid];
      p.o5[(size_t)b * C + h * 64 + j0 + cx.tid] = t;
    }
    bar_sync(BAR_CONS, NCONS);
  }
}

// ------------------------------------------------------------------------------------------------
template <int FMT, int NB, int NT>
__device__ __forceinline__ void consumer(Ctx &cx) {
  const DecodeParams &p = *cx.p;
  for (int pi = 0; pi < p.n_phases; ++pi) {
    const PhaseDev ph = p.phases[pi];
    const bool layered = ph.kind != PH_HEAD && ph.kind != PH_MATVEC;
    const LayerDev *ly = layered ? p.layers + ph.layer : nullptr;
    uint8_t *st0 = p.state + (size_t)(layered ? ph.layer : 0) * p.layer_stride;  // stream 0
    flush_stash(cx);
    switch (ph.kind) {
      case PH_ATT_KVR:
      case PH5_KVRG: {
        const int nvec = p.version == 4 || p.version == 50 ? 3 : 4;
        prologue_ln_mix<NB, NT>(cx, ph.layer == 0, ly->ln1_w, ly->ln1_b, ly->att_mix, nvec, st0);
        cx.stash_dst = st0;
        break;
      }
      case PH_ATT_O:
        if (p.version == 4) prologue_vec<NB, NT>(cx, p.rwkv, p.C);
        else prologue_gn_gate<NB, NT>(cx, *ly);
        break;
      case PH_FFN_KR: {
        const size_t off = p.version == 4 ? (size_t)p.C * act_bytes(p.act_fp16) + 3 * (size_t)p.C * 4
                                          : (size_t)p.C * act_bytes(p.act_fp16) + (size_t)p.H * 4096 * 4;
        prologue_ln_mix<NB, NT>(cx, 0, ly->ln2_w, ly->ln2_b, ly->ffn_mix, 2, st0 + off);
        cx.stash_dst = st0 + off;
        break;
      }
      case PH_FFN_V: prologue_vec<NB, NT>(cx, p.kk, p.F); break;
      case PH_HEAD: prologue_ln_mix<NB, NT>(cx, 0, p.lnout_w, p.lnout_b, nullptr, 0, nullptr); break;
      case PH_MATVEC: prologue_vec<NB, NT>(cx, p.kk, ph.K); break;
      default: break;
    }
    if (ph.kind == PH5_WKV) phase_wkv5(cx, ph, *ly);
    else run_items<FMT, NB, NT>(cx, ph, ly);
    if (pi + 1 < p.n_phases) grid_barrier(cx);
  }
}

template <int FMT>
__device__ __forceinline__ void producer(Ctx &cx) {
  const DecodeParams &p = *cx.p;
  const int KT = kt_max(FMT);
  int slot = 0;
  uint32_t parity = 1;  // a fresh barrier reads as "previous phase complete"
  bool live = true;
  for (int pi = 0; pi < p.n_phases && live; ++pi) {
    const PhaseDev ph = p.phases[pi];
    if (ph.n_items == 0) continue;
    const int nst = num_stages(FMT, ph.K);
    const size_t sub_bytes = rowblock_bytes(FMT, ph.K);
    const size_t item_bytes = sub_bytes * ph.n_sub;
    const int first = (cx.cta + cx.G - ph.rot) % cx.G;
    for (int it = first; it < ph.n_items && live; it += cx.G) {
      const uint8_t *src = ph.w + (size_t)it * item_bytes;
      for (int u = 0; u < ph.n_sub && live; ++u) {
        for (int s = 0; s < nst; ++s) {
          const int kt = min(KT, ph.K - s * KT);
          const uint32_t bytes = stage_bytes(FMT, kt);
          if (!mbar_wait(&cx.sm.empty[slot], parity, cx.sm.abort_flag, p.status, ST_TIMEOUT_EMPTY)) {
            live = false;
            break;
          }
          mbar_expect_tx(&cx.sm.full[slot], bytes);
          bulk_g2s(cx.sm.ring + (size_t)slot * SLOT_BYTES, src, bytes, &cx.sm.full[slot]);
          src += bytes;
          if (++slot == p.n_stages) { slot = 0; parity ^= 1u; }
        }
      }
    }
  }
  if (!live) {
    // give copies that are still in flight time to land before the CTA's shared memory goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
}

template <int FMT, int NB, int NT>
__global__ void __launch_bounds__(NTHREADS, 1) decode_kernel(const __grid_constant__ DecodeParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  Ctx cx;
  cx.p = &p;
  cx.tid = threadIdx.x; cx.warp = threadIdx.x >> 5; cx.lane = threadIdx.x & 31;
  cx.cta = blockIdx.x; cx.G = gridDim.x;
  cx.slot = 0; cx.parity = 0; cx.epoch = 0; cx.stash_dst = nullptr;
  size_t o_stash, o_red, o_xs, o_ring;
  smem_layout<NB, NT>(xs_halfs_needed(p.C, p.F, p.version, NB, NT), p.n_stages, &o_stash, &o_red, &o_xs, &o_ring);
  cx.sm.full = reinterpret_cast<uint64_t *>(smem);
  cx.sm.empty = cx.sm.full + MAX_STAGES;
  cx.sm.abort_flag = reinterpret_cast<volatile int *>(smem + 256);
  cx.sm.ln_red = reinterpret_cast<float *>(smem + 320);
  cx.sm.stats = reinterpret_cast<float *>(smem + 896);
  cx.sm.stash = reinterpret_cast<float *>(smem + o_stash);
  cx.sm.red = reinterpret_cast<float *>(smem + o_red);
  cx.sm.xs = reinterpret_cast<__half *>(smem + o_xs);
  cx.sm.ring = smem + o_ring;
  const int per = (p.C + cx.G - 1) / cx.G;
  cx.own0 = min(cx.cta * per, p.C);
  cx.ownn = min(per, p.C - cx.own0);

  if (cx.tid == 0) {
    for (int s = 0; s < p.n_stages; ++s) {
      mbar_init(&cx.sm.full[s], 1);
      mbar_init(&cx.sm.empty[s], NW);
    }
    *cx.sm.abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (cx.warp == NW) {
    if (cx.lane == 0) producer<FMT>(cx);
  } else {
    consumer<FMT, NB, NT>(cx);
    // last arrival resets the barrier words for the next launch
    bar_sync(BAR_CONS, NCONS);
    if (cx.tid == 0) {
      __threadfence();
      const unsigned done = atomicAdd(p.sync + 1, 1u);
      if (done == (unsigned)cx.G - 1) {
        p.sync[0] = 0;
        p.sync[1] = 0;
        __threadfence();
      }
    }
  }
}

__global__ void argmax_kernel(const float *logits, int V, int Vpad, int32_t *out) {
  const float *row = logits + (size_t)blockIdx.x * Vpad;
  float best = -INFINITY;
  int bi = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; bi = i; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
  }
}

template <int FMT, int NB, int NT>
cudaError_t launch_t(const DecodeParams &p, int grid, size_t smem, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(decode_kernel<FMT, NB, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  void *args[] = {const_cast<DecodeParams *>(&p)};
  return cudaLaunchCooperativeKernel((void *)decode_kernel<FMT, NB, NT>, dim3(grid), dim3(NTHREADS), args, smem, st);
}

template <int FMT, int NB, int NT>
cudaError_t max_grid_t(size_t smem, int device, int *grid) {
  cudaError_t e = cudaFuncSetAttribute(decode_kernel<FMT, NB, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int per_sm = 0, sms = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_kernel<FMT, NB, NT>, NTHREADS, smem);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return e;
  *grid = per_sm > 0 ? sms : 0;
  return cudaSuccess;
}

}  // namespace

// mode: 0 = one stream, 1 = up to 4 streams, 2 = up to 8 streams
size_t decode_smem_bytes(int fmt, int mode, int C, int F, int version, int n_stages) {
  (void)fmt;
  size_t a, b, c, d;
  switch (mode) {
    case 0: return smem_layout<2, 1>(xs_halfs_needed(C, F, version, 2, 1), n_stages, &a, &b, &c, &d);
    case 1: return smem_layout<8, 1>(xs_halfs_needed(C, F, version, 8, 1), n_stages, &a, &b, &c, &d);
    default: return smem_layout<8, 2>(xs_halfs_needed(C, F, version, 8, 2), n_stages, &a, &b, &c, &d);
  }
}

#define FRB_DISPATCH(fn, ...)                                     \
  switch (fmt * 3 + mode) {                                       \
    case 0: return fn<FMT_FP16, 2, 1>(__VA_ARGS__);               \
    case 1: return fn<FMT_FP16, 8, 1>(__VA_ARGS__);               \
    case 2: return fn<FMT_FP16, 8, 2>(__VA_ARGS__);               \
    case 3: return fn<FMT_INT8, 2, 1>(__VA_ARGS__);               \
    case 4: return fn<FMT_INT8, 8, 1>(__VA_ARGS__);               \
    case 5: return fn<FMT_INT8, 8, 2>(__VA_ARGS__);               \
    case 6: return fn<FMT_INT4, 2, 1>(__VA_ARGS__);               \
    case 7: return fn<FMT_INT4, 8, 1>(__VA_ARGS__);               \
    case 8: return fn<FMT_INT4, 8, 2>(__VA_ARGS__);               \
    default: return cudaErrorInvalidValue;                        \
  }

cudaError_t launch_decode(const DecodeParams &p, int mode, int grid, size_t smem, cudaStream_t st) {
  const int fmt = p.fmt;
  FRB_DISPATCH(launch_t, p, grid, smem, st)
}

cudaError_t decode_max_grid(int fmt, int mode, size_t smem, int device, int *grid) {
  FRB_DISPATCH(max_grid_t, smem, device, grid)
}

cudaError_t launch_argmax(const float *logits, int B, int V, int Vpad, int32_t *out, cudaStream_t st) {
  argmax_kernel<<<B, 1024, 0, st>>>(logits, V, Vpad, out);
  return cudaGetLastError();
}

}  // namespace frb
