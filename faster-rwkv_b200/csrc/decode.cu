// Persistent whole-token decode kernel for sm_100a.
//
// One cooperative launch (all CTAs co-resident, one per SM) runs a whole token — all layers and the
// head — for up to 8 independent streams.  Each CTA has one producer warp and NW consumer warps:
//   * the producer walks the CTA's static list of weight tiles (a function of phase index and CTA id
//     only) and keeps a ring of shared-memory stages full with 1-D TMA bulk copies; weights do not
//     depend on activations, so it runs ahead across phase boundaries;
//   * the consumers stage the phase's input vectors in shared memory as fp16 tensor-core operands
//     (LayerNorm + token-shift mix fused here), then for every 16-row block multiply the streamed
//     tile with mma.sync.m16n8k16 (weights = A operand, streams = B operand columns, fp32
//     accumulation, int8/int4 dequantised in registers), reduce across the warps that split K, and
//     apply the phase's epilogue (WKV state update + sigmoid gate, residual add, squared ReLU, ...).
//     Each activation is fed as two fp16 columns, hi = fp16(x) and lo = fp16(x - hi), whose results
//     are added: the operand keeps ~22 mantissa bits at no extra MMA for one stream (7 of the 8
//     columns are idle anyway) and 4 streams share one MMA.
//
// Phases are not separated by barriers.  Every value one phase hands to the next across CTAs is one
// 32-bit word: the fp32 value rounded to 16 significant bits, its low 8 mantissa bits replaced by an
// 8-bit tag of the writing phase; a reader polls the words it needs until they carry the expected tag.  Because each phase needs all outputs of the one before it,
// a CTA can only overwrite a vector after every reader of its previous contents has moved on; a CTA
// that owns no row block in a phase skips the phase.  The token-shift states are double-buffered for
// the same reason.  Every wait is bounded: after WAIT_LIMIT_NS the CTA records a status and drains.
#include "common.cuh"
#include "internal.h"

namespace frb {

namespace {

constexpr int BAR_CONS = 1;  // named barrier id of the consumer warps

struct Smem {
  uint64_t *full, *empty;
  volatile int *abort_flag;
  float *ln_red;     // [NW][2*MAX_B]
  float *red;        // [3][NW][RED_N] per-warp partial sums of the current row block
  float *par;        // one-stream mode: LayerNorm parameters of the next LN phase, staged with bulk copies (or null)
  uint64_t *par_bar; // completion barrier of those copies
  uint64_t *par_free; // consumers -> producer: sm.par may be overwritten
  __half *xs;        // operand vectors
  uint8_t *ring;
};

// NB = operand columns kept per n-tile (2: one stream as hi/lo; 8: four streams as hi/lo), NT = n-tiles.
template <int NB, int NT> __host__ __device__ constexpr int n_streams() { return NB == 2 ? 1 : 4 * NT; }
template <int NB, int NT> __host__ __device__ constexpr int red_n() { return ROWS * n_streams<NB, NT>(); }

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int XR = 2;        // float4 slots per thread that the one-stream LayerNorm keeps in registers
constexpr int PAR_VECS = 7;  // staged per LN phase: gamma, beta, up to 4 mix vectors, the shift state

__host__ __device__ inline size_t xs_halfs_needed(int C, int F, int version, int NB, int NT) {
  size_t a = (size_t)(version == 4 ? 3 : 4) * C;
  size_t b = F;
  return (a > b ? a : b) * NB * NT;
}
// one stream and a model narrow enough for the register-resident LayerNorm: parameters are staged in shared memory,
// as fp16 when every LayerNorm / mix vector of the model is exact in fp16 (a "cuda fp16" file): half the space, which
// buys another ring slot for the weight stream
template <int NB, int NT> __host__ __device__ inline size_t par_bytes(int C, int par16) {
  return (NB == 2 && (C >> 2) <= XR * NCONS) ? (size_t)PAR_VECS * C * (par16 ? 2 : 4) : 0;
}

template <int NB, int NT>
__host__ __device__ inline size_t smem_layout(int fmt, int C, int F, int version, int n_stages, int par16, size_t *off_red,
                                              size_t *off_par, size_t *off_xs, size_t *off_ring) {
  size_t o = 1024;  // barriers + flags + LN scratch
  *off_red = o;   o += sizeof(float) * 3 * NW * red_n<NB, NT>() * (NB == 2 ? 2 : 1);
  o = align_up(o, 128);
  *off_par = o;   o += par_bytes<NB, NT>(C, par16);
  *off_xs = o;    o += xs_halfs_needed(C, F, version, NB, NT) * 2;
  o = align_up(o, 1024);
  *off_ring = o;  o += (size_t)n_stages * slot_bytes(fmt);
  return o;
}

// ------------------------------------------------------------------------------------------------
// stage x operand -> accumulators.  acc[e][t]: two interleaved accumulator sets e (breaks the MMA
// dependency chain), n-tile t.
template <int FMT, int NB, int NT>
__device__ __forceinline__ void process_stage(uint32_t st, int nch, uint32_t xv, uint32_t plane_bytes, int chunk0,
                                              int warp, int lane, float acc[2][NT][4]) {
  const int g = lane >> 2, q = lane & 3;
  const int n = NB == 2 ? (g & 1) : g;   // operand column this lane feeds
  // st, xv: shared-space addresses of the stage and of the operand vector
  for (int c = warp; c < nch; c += NW) {
    const uint32_t xo = xv + ((uint32_t)((chunk0 + c) * 2 * NB + n) * 4u + (uint32_t)q) * 16u;
    uint4 b01[NT], b23[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      b01[t] = lds128(xo + t * plane_bytes);                // MMAs 0,1 of the chunk
      b23[t] = lds128(xo + t * plane_bytes + NB * 4 * 16);  // MMAs 2,3
    }
    if (FMT == FMT_FP16) {
      const uint32_t A = st + (uint32_t)c * 2048u + (uint32_t)lane * 16u;
      const uint4 a0 = lds128(A), a1 = lds128(A + 512), a2 = lds128(A + 1024), a3 = lds128(A + 1536);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        mma16816(acc[0][t], a0.x, a0.y, a0.z, a0.w, b01[t].x, b01[t].y);
        mma16816(acc[1][t], a1.x, a1.y, a1.z, a1.w, b01[t].z, b01[t].w);
        mma16816(acc[0][t], a2.x, a2.y, a2.z, a2.w, b23[t].x, b23[t].y);
        mma16816(acc[1][t], a3.x, a3.y, a3.z, a3.w, b23[t].z, b23[t].w);
      }
    } else if (FMT == FMT_INT8) {
      const uint32_t A = st + (uint32_t)c * 1024u + (uint32_t)lane * 16u;
      const uint4 w01 = lds128(A), w23 = lds128(A + 512);
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
      const uint4 w = lds128(st + (uint32_t)c * 512u + (uint32_t)lane * 16u);
      const uint2 scw = lds64(st + (uint32_t)nch * 512u + (uint32_t)c * 64u + (uint32_t)g * 8u);
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
  uint32_t slot_b;     // bytes per ring slot
  int prof_phase;
  uint32_t red_buf;    // one stream: partial-sum buffer of the next row block (0 / 1)
  bool ready;          // the next stage's tile was seen complete by an earlier look-ahead
  long long pc[5];     // trace: cycle counter at the prologue's milestones (thread 0)
  uint32_t par_parity; // parity of the next wait on sm.par_bar
  unsigned long long wait_ns;  // trace: cycles thread 0 spent waiting for weight tiles in the current phase
};

__device__ __forceinline__ int token_id(const DecodeParams &p, int b) {
  return p.ids_packed ? (int)(0xffffffffu - (unsigned)__ldcg(p.ids_packed + b)) : p.ids_val[b];
}
// 8-bit tag of phase pi of this launch, never 0 (a zeroed buffer matches no phase).  Two consecutive writes of
// one exchange slot are a handful of phases apart, so their tags differ.
__device__ __forceinline__ unsigned phase_tag(const DecodeParams &p, int pi) {
  return 1u + (p.seq_base + (unsigned)pi) % 255u;
}

// ---- tagged exchange words ----------------------------------------------------------------------
// One 32-bit word per value: the fp32 value rounded to 16 significant bits, its low 8 mantissa bits replaced
// by the writer's phase tag.  A reader that sees its tag has the value; no second round trip, no fence.
__device__ __forceinline__ void ex_store(exch_t *dst, float v, unsigned tag) {
  unsigned u = __float_as_uint(v);
  u = ((u & 0x7f800000u) == 0x7f800000u ? u : u + 0x80u) & 0xffffff00u;   // round to nearest; inf / nan keep their class
  asm volatile("st.relaxed.gpu.global.b32 [%0], %1;" ::"l"(dst), "r"(u | tag) : "memory");
}
__device__ __forceinline__ exch_t ex_load_raw(const exch_t *src) {
  exch_t w;
  asm volatile("ld.relaxed.gpu.global.b32 %0, [%1];" : "=r"(w) : "l"(src) : "memory");
  return w;
}
__device__ __forceinline__ float ex_value(exch_t w) { return __uint_as_float(w & 0xffffff00u); }
__device__ __forceinline__ bool ex_ready(exch_t w, unsigned tag) { return (w & 0xffu) == tag; }
// one word; false while the writer has not stored it yet
__device__ __forceinline__ bool ex_try1(const exch_t *src, unsigned tag, float &v) {
  const exch_t w = ex_load_raw(src);
  v = ex_value(w);
  return ex_ready(w, tag);
}
// four consecutive words (16-byte aligned)
__device__ __forceinline__ bool ex_try4(const exch_t *src, unsigned tag, float4 &v) {
  exch_t a, b, c, d;
  asm volatile("ld.relaxed.gpu.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(src) : "memory");
  v = make_float4(ex_value(a), ex_value(b), ex_value(c), ex_value(d));
  // all four tags equal `tag`: compare the tag bytes in one go
  return ((a & 0xffu) | ((b & 0xffu) << 8) | ((c & 0xffu) << 16) | (d << 24)) == tag * 0x01010101u;
}

__device__ __forceinline__ uint4 ex_load_raw4(const exch_t *src) {
  uint4 w;
  asm volatile("ld.relaxed.gpu.global.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src) : "memory");
  return w;
}
__device__ __forceinline__ bool ex_decode4(const uint4 &w, unsigned tag, float4 &v) {
  v = make_float4(ex_value(w.x), ex_value(w.y), ex_value(w.z), ex_value(w.w));
  return ((w.x & 0xffu) | ((w.y & 0xffu) << 8) | ((w.z & 0xffu) << 16) | (w.w << 24)) == tag * 0x01010101u;
}

// Bounded polling: gives up after WAIT_LIMIT_NS (or as soon as another thread of the CTA gave up).
struct Poll {
  unsigned long long t0;
  int it;
  __device__ __forceinline__ Poll() : t0(0), it(0) {}
  __device__ __forceinline__ bool keep_waiting(Ctx &cx) {
    if ((++it & 63) != 0) return true;
    if (*cx.sm.abort_flag) return false;
    const unsigned long long now = globaltimer_ns();
    if (t0 == 0) t0 = now;
    if (now - t0 > WAIT_LIMIT_NS || __ldcg(cx.p->status) != 0) {
      *cx.sm.abort_flag = 1;
      atomicCAS(cx.p->status, 0, ST_TIMEOUT_DATA + 1000 * cx.prof_phase);   // which phase gave up
      return false;
    }
    return true;
  }
};
__device__ __forceinline__ float ex_wait1(Ctx &cx, const exch_t *src, unsigned tag) {
  float v;
  Poll poll;
  while (!ex_try1(src, tag, v) && poll.keep_waiting(cx)) { }
  return v;
}
__device__ __forceinline__ float4 ex_wait4(Ctx &cx, const exch_t *src, unsigned tag) {
  float4 v;
  Poll poll;
  while (!ex_try4(src, tag, v) && poll.keep_waiting(cx)) { }
  return v;
}

// Wait until an exchange vector [B][K] written by phase `tag` is (almost certainly) complete, touching as
// little of it as possible: writers store 16 consecutive words (one row block) with one warp instruction,
// so polling the first word of every block tells when the block has landed.  The full read that follows
// still checks every tag.  Keeps 148 CTAs from hammering the whole vector while they wait.
template <int SB>
__device__ __forceinline__ void wait_sentinels(Ctx &cx, const exch_t *src, int K, unsigned tag) {
  const int per = K / ROWS, n = cx.p->B * per;
  constexpr int SR = 8;   // sentinels asked for together: one round trip, then the tags are looked at
  Poll poll;
  bool ok;
  if constexpr (SB == 1) {   // a few words per thread: the plain sweep is the faster one (measured)
    do {
      ok = true;
      for (int idx = cx.tid; idx < n; idx += NCONS) {
        float v;
        ok = ex_try1(src + (size_t)idx * ROWS, tag, v) && ok;
      }
    } while (!ok && poll.keep_waiting(cx));
  } else {
  do {
    ok = true;
    for (int base = cx.tid; base < n; base += SR * NCONS) {
      exch_t w[SR];
#pragma unroll
      for (int r = 0; r < SR; ++r) {
        const int idx = base + r * NCONS;
        if (idx < n) {
          const int b = idx / per, t = idx - b * per;
          w[r] = ex_load_raw(src + (size_t)b * K + (size_t)t * ROWS);
        }
      }
#pragma unroll
      for (int r = 0; r < SR; ++r)
        if (base + r * NCONS < n) ok = ex_ready(w[r], tag) && ok;
    }
  } while (!ok && poll.keep_waiting(cx));
  }
  bar_sync(BAR_CONS, NCONS);
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
__device__ __forceinline__ void store_act4(uint8_t *base, int i4, int act_fp16, const float4 &v) {
  if (act_fp16) {
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t *>(&lo);
    u.y = *reinterpret_cast<const uint32_t *>(&hi);
    reinterpret_cast<uint2 *>(base)[i4] = u;
  } else {
    reinterpret_cast<float4 *>(base)[i4] = v;
  }
}

// Operand position of stream b inside a vector: n-tile plane and the hi / lo columns.
template <int NB>
__device__ __forceinline__ void operand_cols(int b, int &tile, int &col_hi, int &col_lo) {
  if (NB == 2) { tile = 0; col_hi = 0; col_lo = 1; }
  else { tile = b >> 2; col_hi = b & 3; col_lo = 4 + (b & 3); }
}

// Write 4 consecutive inputs k..k+3 of stream b into operand vector `vec` as hi + lo fp16 columns.
// Every lane of the warp must make the call (`valid` says whether this lane has data), with k = 4 * i4 and
// i4 = lane (mod 8).  One stream: the lane pair (l, l ^ 4) holds the even and the odd 16-input group of a
// 32-input block; they swap halves so that one lane stores the 16 hi bytes and the other the 16 lo bytes, and a
// quarter warp writes 128 contiguous bytes (no bank conflicts).
template <int NB>
__device__ __forceinline__ void store_operand4(__half *vec, size_t plane_halfs, int k, int b, float a, float bb, float c,
                                               float dd, bool valid) {
  const __half2 h0 = __floats2half2_rn(a, bb), h1 = __floats2half2_rn(c, dd);
  const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
  const __half2 l0 = __floats2half2_rn(a - f0.x, bb - f0.y), l1 = __floats2half2_rn(c - f1.x, dd - f1.y);
  const uint32_t uh0 = *reinterpret_cast<const uint32_t *>(&h0), uh1 = *reinterpret_cast<const uint32_t *>(&h1);
  const uint32_t ul0 = *reinterpret_cast<const uint32_t *>(&l0), ul1 = *reinterpret_cast<const uint32_t *>(&l1);
  if (NB == 2) {
    const bool odd = (k >> 4) & 1;
    const uint32_t rx = __shfl_xor_sync(0xffffffffu, odd ? uh0 : ul0, 4);
    const uint32_t ry = __shfl_xor_sync(0xffffffffu, odd ? uh1 : ul1, 4);
    const uint4 u = odd ? make_uint4(rx, ry, ul0, ul1) : make_uint4(uh0, uh1, rx, ry);
    if (valid) *reinterpret_cast<uint4 *>(vec + xs_index(k & ~16, odd ? 1 : 0, NB)) = u;
  } else if (valid) {
    int tile, ch, cl;
    operand_cols<NB>(b, tile, ch, cl);
    __half *pl = vec + (size_t)tile * plane_halfs;
    *reinterpret_cast<uint2 *>(pl + xs_index(k, ch, NB)) = make_uint2(uh0, uh1);
    *reinterpret_cast<uint2 *>(pl + xs_index(k, cl, NB)) = make_uint2(ul0, ul1);
  }
}

// Element 4*i4.. of the residual stream of stream b without waiting: the embedding row at layer 0
// (always there), else one attempt at the tagged words.
__device__ __forceinline__ bool try_x4(const DecodeParams &p, const exch_t *xsrc, bool layer0, int b, int i4, unsigned tag, float4 &v) {
  if (layer0) {
    if (p.emb_f32) {
      v = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.emb) + (size_t)token_id(p, b) * p.C) + i4);
    } else {
      const __half *row = reinterpret_cast<const __half *>(p.emb) + (size_t)token_id(p, b) * p.C;
      const uint2 u = __ldg(reinterpret_cast<const uint2 *>(row) + i4);
      const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
      const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
      v = make_float4(a.x, a.y, c.x, c.y);
    }
    return true;
  }
  return ex_try4(xsrc + (size_t)b * p.C + (size_t)i4 * 4, tag, v);
}

// Normalised value -> operand vectors (token-shift mix) and, on the owning CTA, the new shift state.
template <int NB, int NT>
__device__ __forceinline__ void ln_emit(Ctx &cx, const PhaseDev &ph, int nvec, uint8_t *sx_wr, int sx_item0, int i4, int b,
                                        const float4 &xv, float mean, float rstd, const float4 &gw, const float4 &gb,
                                        const float4 *mx4, const float4 &sx, bool valid) {
  const DecodeParams &p = *cx.p;
  const size_t plane = (size_t)p.C * NB;   // halfs per (vector, n-tile)
  const size_t vstride = plane * NT;       // halfs per operand vector
  float4 xx;
  xx.x = (xv.x - mean) * rstd * gw.x + gb.x;
  xx.y = (xv.y - mean) * rstd * gw.y + gb.y;
  xx.z = (xv.z - mean) * rstd * gw.z + gb.z;
  xx.w = (xv.w - mean) * rstd * gw.w + gb.w;
  if (nvec == 0) {
    store_operand4<NB>(cx.sm.xs, plane, i4 * 4, b, xx.x, xx.y, xx.z, xx.w, valid);
    return;
  }
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (v < nvec) {
      const float4 m = mx4[v];
      store_operand4<NB>(cx.sm.xs + v * vstride, plane, i4 * 4, b, xx.x * m.x + sx.x * (1.f - m.x),
                         xx.y * m.y + sx.y * (1.f - m.y), xx.z * m.z + sx.z * (1.f - m.z),
                         xx.w * m.w + sx.w * (1.f - m.w), valid);
    }
  }
  // new token-shift state: written once, by the CTA that owns the row block of these channels
  if (valid && (sx_item0 + (i4 >> 2) + ph.rot) % cx.G == cx.cta)
    store_act4(sx_wr + (size_t)b * p.state_stride, i4, p.act_fp16, xx);
}

// What a LayerNorm phase reads besides the residual stream.
struct LnArgs {
  const exch_t *xsrc;   // residual stream this LayerNorm reads
  const float *ln_w, *ln_b;
  const float *const *mix;
  const uint8_t *sx_rd;
  uint8_t *sx_wr;
  int nvec, item0;
  bool layer0;
};
__device__ __forceinline__ bool is_ln_phase(int kind) {
  return kind == PH_ATT_KVR || kind == PH5_KVRG || kind == PH_FFN_KR || kind == PH_HEAD;
}
__device__ __forceinline__ LnArgs ln_args(const DecodeParams &p, const PhaseDev &ph) {
  LnArgs a;
  const int v5 = p.version != 4, par = (int)(p.par_mask & 1u);   // streams of one launch share the parity
  a.ln_w = p.lnout_w; a.ln_b = p.lnout_b; a.mix = nullptr; a.sx_rd = nullptr; a.sx_wr = nullptr;
  a.nvec = 0; a.item0 = 0; a.layer0 = false; a.xsrc = p.x;
  if (ph.kind == PH_HEAD) return a;
  const LayerDev *ly = p.layers + ph.layer;
  uint8_t *st0 = p.state + (size_t)ph.layer * p.layer_stride;   // stream 0
  if (ph.kind == PH_FFN_KR) {
    a.ln_w = ly->ln2_w; a.ln_b = ly->ln2_b; a.mix = ly->ffn_mix; a.nvec = 2; a.item0 = ph.split[0]; a.xsrc = p.xa;
    a.sx_rd = st0 + off_ffn_sx(p.C, p.H, v5, p.act_fp16, par);
    a.sx_wr = st0 + off_ffn_sx(p.C, p.H, v5, p.act_fp16, par ^ 1);
  } else {
    a.ln_w = ly->ln1_w; a.ln_b = ly->ln1_b; a.mix = ly->att_mix;
    a.nvec = p.version == 4 || p.version == 50 ? 3 : 4;
    a.sx_rd = st0 + off_sx(p.C, p.act_fp16, par);
    a.sx_wr = st0 + off_sx(p.C, p.act_fp16, par ^ 1);
    a.layer0 = ph.layer == 0;
  }
  return a;
}

// Copy an LN phase's parameters (and shift state) into sm.par: one bulk copy per vector, all completing on
// sm.par_bar.  Issued by the producer thread when it reaches the phase's first weight tile, which is a ring depth
// ahead of the consumers; the LayerNorm prologue waits on the barrier.
__device__ __forceinline__ void ln_stage_params(Ctx &cx, const LnArgs &a) {
  const DecodeParams &p = *cx.p;
  uint8_t *par = reinterpret_cast<uint8_t *>(cx.sm.par);
  const uint32_t vb = (uint32_t)p.C * (p.vecs16 ? 2u : 4u);   // bytes per staged vector
  const uint32_t sxb = a.nvec > 0 ? (uint32_t)p.C * (p.act_fp16 ? 2u : 4u) : 0u;
  // the fp16 image of a vector sits at the same element offset in the fp16 copy of the vector blob
  auto src = [&](const float *v) -> const void * {
    return p.vecs16 ? static_cast<const void *>(p.vecs16 + (v - p.vecs32)) : static_cast<const void *>(v);
  };
  mbar_expect_tx(cx.sm.par_bar, vb * (2u + (uint32_t)a.nvec) + sxb);
  bulk_g2s(par, src(a.ln_w), vb, cx.sm.par_bar);
  bulk_g2s(par + vb, src(a.ln_b), vb, cx.sm.par_bar);
  for (int v = 0; v < a.nvec; ++v) bulk_g2s(par + (2 + v) * vb, src(a.mix[v]), vb, cx.sm.par_bar);
  if (a.nvec > 0) bulk_g2s(par + 6 * vb, a.sx_rd, sxb, cx.sm.par_bar);
}

// LayerNorm + token-shift mix for ONE stream of a model with n_embd <= 4 * XR * NCONS: the latency-critical
// prologue of batch-1 decode.  The parameters were staged into shared memory ahead of time (ln_stage_params), so
// the only global round trip left is the one that fetches x: every thread polls its own slots plus the pivot
// element together until all tags match.  Statistics: shifted single pass, sums of (x - x[0]) and (x - x[0])^2.
// nvec == 0: plain LayerNorm -> operand vector 0 (head).
template <int NB, int NT>
__device__ __forceinline__ void prologue_ln_one(Ctx &cx, const PhaseDev &ph, const LnArgs &a, unsigned xtag) {
  const DecodeParams &p = *cx.p;
  const int n4 = p.C >> 2;
  float4 xv[XR], pv;
  Poll poll;
  unsigned pending = 1u << XR;   // bit XR: the pivot; bits 0..XR-1: this thread's slots still missing
#pragma unroll
  for (int r = 0; r < XR; ++r)
    if (cx.tid + r * NCONS < n4) pending |= 1u << r;
  do {
    if ((pending >> XR) && try_x4(p, a.xsrc, a.layer0, 0, 0, xtag, pv)) pending &= ~(1u << XR);
#pragma unroll
    for (int r = 0; r < XR; ++r)
      if ((pending & (1u << r)) && try_x4(p, a.xsrc, a.layer0, 0, cx.tid + r * NCONS, xtag, xv[r])) pending &= ~(1u << r);
  } while (pending && poll.keep_waiting(cx));
  if (p.prof && cx.tid == 0) cx.pc[2] = clock64();  // trace
  const float piv = pv.x;
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int r = 0; r < XR; ++r) {
    const int i4 = cx.tid + r * NCONS;
    if (i4 < n4) {
      const float d0 = xv[r].x - piv, d1 = xv[r].y - piv, d2 = xv[r].z - piv, d3 = xv[r].w - piv;
      s1 += (d0 + d1) + (d2 + d3);
      s2 += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
  }
  if (cx.lane == 0) { cx.sm.ln_red[cx.warp * 2] = s1; cx.sm.ln_red[cx.warp * 2 + 1] = s2; }
  mbar_wait(cx.sm.par_bar, cx.par_parity, cx.sm.abort_flag, p.status, ST_TIMEOUT_FULL);   // staged parameters have landed
  cx.par_parity ^= 1u;
  bar_sync(BAR_CONS, NCONS);
  float sa = 0.f, sc = 0.f;
#pragma unroll
  for (int w = 0; w < NW; ++w) { sa += cx.sm.ln_red[w * 2]; sc += cx.sm.ln_red[w * 2 + 1]; }
  const float inv = 1.f / (float)p.C;
  const float m = sa * inv;
  float var = sc * inv - m * m;
  var = var > 0.f ? var : 0.f;
  const float mean = piv + m, rstd = rsqrtf(var + 1e-5f);
  if (p.prof && cx.tid == 0) cx.pc[3] = clock64();  // trace
  const uint8_t *par = reinterpret_cast<const uint8_t *>(cx.sm.par);
  const bool par16 = p.vecs16 != nullptr;
  const uint32_t vb = (uint32_t)p.C * (par16 ? 2u : 4u);
  auto half4 = [](const uint8_t *base, int i4) {
    const uint2 u = *reinterpret_cast<const uint2 *>(base + (size_t)i4 * 8);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  };
  auto par4 = [&](int v, int i4) {
    return par16 ? half4(par + v * vb, i4) : *reinterpret_cast<const float4 *>(par + v * vb + (size_t)i4 * 16);
  };
#pragma unroll
  for (int r = 0; r < XR; ++r) {
    const bool valid = cx.tid + r * NCONS < n4;
    const int i4 = valid ? cx.tid + r * NCONS : cx.lane & 7;   // lanes without data still make the (warp-wide) call
    if (r * NCONS + (cx.tid & ~31) < n4) {                      // warp-uniform
      const float4 gw = par4(0, i4);
      const float4 gb = par4(1, i4);
      float4 mx4[4], sx = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int v = 0; v < 4; ++v)
        if (v < a.nvec) mx4[v] = par4(2 + v, i4);
      if (a.nvec > 0) sx = p.act_fp16 ? half4(par + 6 * vb, i4) : *reinterpret_cast<const float4 *>(par + 6 * vb + (size_t)i4 * 16);
      ln_emit<NB, NT>(cx, ph, a.nvec, a.sx_wr, a.item0, i4, 0, xv[r], mean, rstd, gw, gb, mx4, sx, valid);
    }
  }
  __syncwarp();
  if (cx.lane == 0) mbar_arrive(cx.sm.par_free);   // this warp is done with sm.par: the producer may refill it
  bar_sync(BAR_CONS, NCONS);
  if (p.prof && cx.tid == 0) cx.pc[4] = clock64();  // trace
}

// LayerNorm + token-shift mix, any number of streams and any width: a statistics pass (which also waits for the
// data) and a second pass over x.  Every CTA needs the whole operand of every stream, so the prologue's length is
// the number of dependent round trips to L2 it makes: each pass asks for the words of all streams and of all its
// slots (and the second one for the parameters and shift states as well) before it looks at any of them; with up
// to four streams of a model that fits the slots, x stays in registers between the passes.
// x[b][4 * i4s[j] ..] for every stream b < B and every used slot j, all requested before any is examined; words that
// have not arrived are asked for again (bounded like every wait)
template <int SB, int JB>
__device__ __forceinline__ void batch_x4(Ctx &cx, const exch_t *xsrc, bool layer0, unsigned tag, const int (&i4s)[JB],
                                         const bool (&use)[JB], float4 (&v)[SB][JB]) {
  const DecodeParams &p = *cx.p;
  if (layer0) {   // embedding rows: plain loads, always there
#pragma unroll
    for (int b = 0; b < SB; ++b)
#pragma unroll
      for (int j = 0; j < JB; ++j)
        if (b < p.B && use[j]) try_x4(p, xsrc, true, b, i4s[j], tag, v[b][j]);
    return;
  }
  unsigned pending = 0;
#pragma unroll
  for (int b = 0; b < SB; ++b)
#pragma unroll
    for (int j = 0; j < JB; ++j)
      if (b < p.B && use[j]) pending |= 1u << (b * JB + j);
  Poll poll;
  while (pending) {
    // the raw words land in v itself and are decoded in place: no second set of registers
#pragma unroll
    for (int b = 0; b < SB; ++b)
#pragma unroll
      for (int j = 0; j < JB; ++j)
        if ((pending >> (b * JB + j)) & 1u) {
          const uint4 w = ex_load_raw4(xsrc + (size_t)b * p.C + (size_t)i4s[j] * 4);
          v[b][j] = make_float4(__uint_as_float(w.x), __uint_as_float(w.y), __uint_as_float(w.z), __uint_as_float(w.w));
        }
#pragma unroll
    for (int b = 0; b < SB; ++b)
#pragma unroll
      for (int j = 0; j < JB; ++j)
        if ((pending >> (b * JB + j)) & 1u) {
          const uint4 w = make_uint4(__float_as_uint(v[b][j].x), __float_as_uint(v[b][j].y), __float_as_uint(v[b][j].z),
                                     __float_as_uint(v[b][j].w));
          float4 t;
          if (ex_decode4(w, tag, t)) { v[b][j] = t; pending &= ~(1u << (b * JB + j)); }
        }
    if (pending && !poll.keep_waiting(cx)) break;
  }
}

template <int NB, int NT>
__device__ __forceinline__ void prologue_ln_mix(Ctx &cx, const PhaseDev &ph, const exch_t *xsrc, bool layer0, unsigned xtag, const float *ln_w,
                                             const float *ln_b, const float *const *mix, int nvec, const uint8_t *sx_rd,
                                             uint8_t *sx_wr, int sx_item0) {
  constexpr int SB = n_streams<NB, NT>();
  constexpr int JB = SB > 4 ? 1 : 2;   // slots per thread and round: SB x JB 16-byte loads in flight
  const DecodeParams &p = *cx.p;
  const int n4 = p.C >> 2;
  const float inv = 1.f / (float)p.C;
  const bool fits = n4 <= JB * NCONS;   // one round covers the vector: x stays in registers
  if (!layer0) wait_sentinels<SB>(cx, xsrc, p.C, xtag);
  float s1[SB], s2[SB], piv[SB], mean[SB], rstd[SB];
  float4 xv[SB][JB];
  {
    const int i0[JB] = {};
    bool u0[JB] = {};
    u0[0] = true;
    float4 pv[SB][JB];
    batch_x4<SB, JB>(cx, xsrc, layer0, xtag, i0, u0, pv);
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      s1[b] = s2[b] = 0.f;
      piv[b] = b < p.B ? pv[b][0].x : 0.f;
    }
  }
  for (int base = 0; base < n4; base += JB * NCONS) {
    int i4s[JB];
    bool use[JB];
#pragma unroll
    for (int j = 0; j < JB; ++j) {
      i4s[j] = base + j * NCONS + cx.tid;
      use[j] = i4s[j] < n4;
    }
    batch_x4<SB, JB>(cx, xsrc, layer0, xtag, i4s, use, xv);
#pragma unroll
    for (int b = 0; b < SB; ++b)
#pragma unroll
      for (int j = 0; j < JB; ++j)
        if (b < p.B && use[j]) {
          const float4 v = xv[b][j];
          const float d0 = v.x - piv[b], d1 = v.y - piv[b], d2 = v.z - piv[b], d3 = v.w - piv[b];
          s1[b] += (d0 + d1) + (d2 + d3);
          s2[b] += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        }
  }
#pragma unroll
  for (int b = 0; b < SB; ++b) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s1[b] += __shfl_xor_sync(0xffffffffu, s1[b], o);
      s2[b] += __shfl_xor_sync(0xffffffffu, s2[b], o);
    }
  }
  if (cx.lane == 0) {
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      cx.sm.ln_red[cx.warp * 2 * MAX_B + 2 * b] = s1[b];
      cx.sm.ln_red[cx.warp * 2 * MAX_B + 2 * b + 1] = s2[b];
    }
  }
  bar_sync(BAR_CONS, NCONS);
#pragma unroll
  for (int b = 0; b < SB; ++b) {
    float a = 0.f, c = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      a += cx.sm.ln_red[w * 2 * MAX_B + 2 * b];
      c += cx.sm.ln_red[w * 2 * MAX_B + 2 * b + 1];
    }
    const float m = a * inv;
    float var = c * inv - m * m;
    var = var > 0.f ? var : 0.f;
    mean[b] = piv[b] + m;
    rstd[b] = rsqrtf(var + 1e-5f);
  }
  for (int base = 0; base < n4; base += JB * NCONS) {
    // every lane of a warp that has any data makes the calls (the operand stores may shuffle); lanes past the end
    // work on a dummy index and store nothing
    int i4s[JB];
    bool use[JB], valid[JB];
#pragma unroll
    for (int j = 0; j < JB; ++j) {
      const int i4 = base + j * NCONS + cx.tid;
      use[j] = base + j * NCONS + (cx.tid & ~31) < n4;   // warp-uniform
      valid[j] = i4 < n4;
      i4s[j] = valid[j] ? i4 : cx.lane & 7;
    }
    if (!fits) batch_x4<SB, JB>(cx, xsrc, layer0, xtag, i4s, use, xv);   // already there: the statistics pass waited
#pragma unroll
    for (int j = 0; j < JB; ++j) {
      if (!use[j]) continue;
      // one round trip for this slot's parameters and every stream's shift state
      float4 mx4[4], sxv[SB];
      const float4 gw = __ldg(reinterpret_cast<const float4 *>(ln_w) + i4s[j]);
      const float4 gb = __ldg(reinterpret_cast<const float4 *>(ln_b) + i4s[j]);
#pragma unroll
      for (int v = 0; v < 4; ++v)
        if (v < nvec) mx4[v] = __ldg(reinterpret_cast<const float4 *>(mix[v]) + i4s[j]);
#pragma unroll
      for (int b = 0; b < SB; ++b) {
        sxv[b] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < p.B && nvec > 0) sxv[b] = load_act4(sx_rd + (size_t)b * p.state_stride, i4s[j], p.act_fp16);
      }
#pragma unroll
      for (int b = 0; b < SB; ++b) {
        if (b >= p.B) break;
        ln_emit<NB, NT>(cx, ph, nvec, sx_wr, sx_item0, i4s[j], b, xv[b][j], mean[b], rstd[b], gw, gb, mx4, sxv[b], valid[j]);
      }
    }
  }
  bar_sync(BAR_CONS, NCONS);
}

template <int NB, int NT>
__device__ __forceinline__ void prologue_ln(Ctx &cx, const PhaseDev &ph, int pi, unsigned xtag) {
  const LnArgs a = ln_args(*cx.p, ph);
  if (cx.sm.par) {
    prologue_ln_one<NB, NT>(cx, ph, a, xtag);
  } else {
    prologue_ln_mix<NB, NT>(cx, ph, a.xsrc, a.layer0, xtag, a.ln_w, a.ln_b, a.mix, a.nvec, a.sx_rd, a.sx_wr, a.item0);
  }
}

// exchange vector [B][K] written by phase `tag` -> operand vector 0.  Short vectors are polled directly,
// every thread issuing the loads of all its slots before it looks at a tag; long ones wait on the block
// sentinels first so that the waiting CTAs do not sweep 64 KB each per round.
template <int NB, int NT>
__device__ __forceinline__ void prologue_vec(Ctx &cx, const exch_t *src, int K, unsigned tag) {
  constexpr int SB = n_streams<NB, NT>();
  constexpr int VR = SB == 1 ? 8 : 4;   // slots polled together
  const DecodeParams &p = *cx.p;
  const int n4 = K >> 2;
  const size_t plane = (size_t)K * NB;
  if ((long long)n4 * p.B > (long long)VR * NCONS) wait_sentinels<SB>(cx, src, K, tag);
  const int total = n4 * p.B;   // slot index s -> stream s / n4, float4 s % n4
  for (int base = cx.tid; (base & ~31) < total; base += VR * NCONS) {   // warp-uniform: the stores below shuffle
    float4 v[VR];
    Poll poll;
    unsigned pending = 0;   // slots whose words have not all arrived: only those are asked for again
#pragma unroll
    for (int r = 0; r < VR; ++r)
      if (base + r * NCONS < total) pending |= 1u << r;
    if constexpr (SB == 1) {   // one stream: the compiler keeps these eight requests in flight together as written (measured)
      do {
#pragma unroll
        for (int r = 0; r < VR; ++r) {
          if (pending & (1u << r)) {
            const int s = base + r * NCONS;
            if (ex_try4(src + (size_t)s * 4, tag, v[r])) pending &= ~(1u << r);
          }
        }
      } while (pending && poll.keep_waiting(cx));
    } else {
    while (pending) {
      // all pending slots are requested before any tag is looked at; the raw words land in v and are decoded in place
#pragma unroll
      for (int r = 0; r < VR; ++r) {
        if (pending & (1u << r)) {
          const int s = base + r * NCONS;
          const int b = s / n4, i4 = s - b * n4;
          const uint4 w = ex_load_raw4(src + (size_t)b * K + (size_t)i4 * 4);
          v[r] = make_float4(__uint_as_float(w.x), __uint_as_float(w.y), __uint_as_float(w.z), __uint_as_float(w.w));
        }
      }
#pragma unroll
      for (int r = 0; r < VR; ++r) {
        if (pending & (1u << r)) {
          const uint4 w = make_uint4(__float_as_uint(v[r].x), __float_as_uint(v[r].y), __float_as_uint(v[r].z), __float_as_uint(v[r].w));
          float4 t;
          if (ex_decode4(w, tag, t)) { v[r] = t; pending &= ~(1u << r); }
        }
      }
      if (pending && !poll.keep_waiting(cx)) break;
    }
    }
    if (p.prof && cx.tid == 0) cx.pc[2] = clock64();  // trace
#pragma unroll
    for (int r = 0; r < VR; ++r) {
      const int s = base + r * NCONS;
      if ((s & ~31) < total) {   // warp-uniform
        const bool valid = s < total;
        const int sc = valid ? s : cx.lane & 7;
        const int b = sc / n4, i4 = sc - b * n4;
        store_operand4<NB>(cx.sm.xs, plane, i4 * 4, b, v[r].x, v[r].y, v[r].z, v[r].w, valid);
      }
    }
  }
  if (p.prof && cx.tid == 0) cx.pc[3] = clock64();  // trace
  bar_sync(BAR_CONS, NCONS);
  if (p.prof && cx.tid == 0) cx.pc[4] = clock64();  // trace
}

// plain fp32 vector [B][K] (stand-alone matvec) -> operand vector 0
template <int NB, int NT>
__device__ __forceinline__ void prologue_plain(Ctx &cx, const float *src, int K) {
  constexpr int SB = n_streams<NB, NT>();
  const DecodeParams &p = *cx.p;
  const int n4 = K >> 2;
  const size_t plane = (size_t)K * NB;
  for (int base = 0; base < n4; base += NCONS) {
    if (base + (cx.tid & ~31) >= n4) break;   // warp-uniform
    const bool valid = base + cx.tid < n4;
    const int i4 = valid ? base + cx.tid : cx.lane & 7;
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      if (b >= p.B) break;
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)b * K) + i4);
      store_operand4<NB>(cx.sm.xs, plane, i4 * 4, b, v.x, v.y, v.z, v.w, valid);
    }
  }
  bar_sync(BAR_CONS, NCONS);
}

// v5 output projection input: GroupNorm over each head's 64 readout values, times the gate
template <int NB, int NT>
__device__ __forceinline__ void prologue_gn_gate(Ctx &cx, const PhaseDev &ph, unsigned otag, unsigned gtag) {
  constexpr int SB = n_streams<NB, NT>();
  const DecodeParams &p = *cx.p;
  const size_t plane = (size_t)p.C * NB;
  const int n4 = p.C >> 2;  // 16 float4 per head -> 16 consecutive threads share a head
  wait_sentinels<n_streams<NB, NT>()>(cx, p.o5, p.C, otag);
  for (int base = 0; base < n4; base += NCONS) {
    const int i4 = base + cx.tid;
    const bool ok = i4 < n4;
#pragma unroll
    for (int b = 0; b < SB; ++b) {
      if (b >= p.B) break;
      // the readout, the gate and the GroupNorm parameters are requested together; what has not arrived is waited
      // for afterwards
      float4 v = make_float4(0, 0, 0, 0), gw = v, gb = v, g = v;
      if (ok) {
        const exch_t *op = p.o5 + (size_t)b * p.C + (size_t)i4 * 4, *gp = p.g5 + (size_t)b * p.C + (size_t)i4 * 4;
        const uint4 ow = ex_load_raw4(op);
        uint4 gwd = make_uint4(0u, 0u, 0u, 0u);
        if (p.version >= 51) gwd = ex_load_raw4(gp);
        gw = __ldg(reinterpret_cast<const float4 *>(ph.aux0) + i4);
        gb = __ldg(reinterpret_cast<const float4 *>(ph.aux1) + i4);
        if (!ex_decode4(ow, otag, v)) v = ex_wait4(cx, op, otag);
        if (p.version >= 51 && !ex_decode4(gwd, gtag, g)) g = ex_wait4(cx, gp, gtag);
      }
      float s = (v.x + v.y) + (v.z + v.w);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s * (1.f / 64.f);
      const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
      float q = (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
      const float rstd = rsqrtf(q * (1.f / 64.f) + 1e-5f);
      float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ok) {
        y = make_float4(d0 * rstd * gw.x + gb.x, d1 * rstd * gw.y + gb.y, d2 * rstd * gw.z + gb.z,
                        d3 * rstd * gw.w + gb.w);
        if (p.version >= 51) { y.x *= g.x; y.y *= g.y; y.z *= g.z; y.w *= g.w; }
      }
      store_operand4<NB>(cx.sm.xs, plane, (ok ? i4 : cx.lane & 7) * 4, b, y.x, y.y, y.z, y.w, ok);
    }
  }
  bar_sync(BAR_CONS, NCONS);
}

// ---- epilogue of one (row, stream) output --------------------------------------------------------
// Values the epilogue needs from global memory; requested when the row block starts so that their
// latency hides behind the wait for the weight tiles.
struct EpiIn {
  float a, b, c, d, e;
  exch_t wa, wb;     // exchange words requested early; their tags are checked when the epilogue uses them
  float rscale[3];
};

template <int FMT>
__device__ __forceinline__ void epilogue_prefetch(Ctx &cx, const PhaseDev &ph, int pi, int it, int row,
                                                  int b, EpiIn &in) {
  const DecodeParams &p = *cx.p;
  const int C = p.C;
  if (FMT == FMT_INT8) {
#pragma unroll
    for (int u = 0; u < 3; ++u)
      if (u < ph.n_sub) in.rscale[u] = __half2float(__ldg(ph.rscale + ((size_t)it * ph.n_sub + u) * ROWS + row));
  }
  switch (ph.kind) {
    case PH_ATT_KVR: {
      const int c = it * ROWS + row;
      const uint8_t *st = p.state + (size_t)b * p.state_stride + (size_t)ph.layer * p.layer_stride;
      const float *aa = reinterpret_cast<const float *>(st + off_mid(C, p.act_fp16));
      in.a = aa[c]; in.b = aa[C + c]; in.c = aa[2 * C + c];
      in.d = __ldg(ph.aux0 + c); in.e = __ldg(ph.aux1 + c);
      break;
    }
    case PH_ATT_O: {
      // residual input: the embedding row at layer 0, else x as the previous layer's ffn value phase left it
      const int c = it * ROWS + row;
      if (ph.layer == 0)
        in.a = p.emb_f32 ? __ldg(reinterpret_cast<const float *>(p.emb) + (size_t)token_id(p, b) * C + c)
                         : __half2float(reinterpret_cast<const __half *>(p.emb)[(size_t)token_id(p, b) * C + c]);
      else in.wa = ex_load_raw(p.x + (size_t)b * C + c);
      break;
    }
    case PH_FFN_V: {
      const int c = it * ROWS + row;
      in.wa = ex_load_raw(p.xa + (size_t)b * C + c);   // written by the output projection
      in.wb = ex_load_raw(p.rr + (size_t)b * C + c);   // written by the ffn receptance rows of the phase before
      break;
    }
    default: break;
  }
}

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// value of an exchange word that was requested early: taken if its tag is there, else waited for
__device__ __forceinline__ float ex_finish(Ctx &cx, exch_t w, const exch_t *src, unsigned tag) {
  return ex_ready(w, tag) ? ex_value(w) : ex_wait1(cx, src, tag);
}

__device__ __forceinline__ void epilogue(Ctx &cx, const PhaseDev &ph, int pi, unsigned tag, int it, int row, int b,
                                         const float val[3], const EpiIn &in) {
  const DecodeParams &p = *cx.p;
  const int C = p.C;
  switch (ph.kind) {
    case PH_ATT_KVR: {
      const int c = it * ROWS + row;
      uint8_t *st = p.state + (size_t)b * p.state_stride + (size_t)ph.layer * p.layer_stride;
      float *aa = reinterpret_cast<float *>(st + off_mid(C, p.act_fp16));
      float *bb = aa + C, *pp = bb + C;
      const float k = val[0], v = val[1], r = sigmoid_f(val[2]);
      const float u = in.d, w = in.e;
      const float a0 = in.a, b0 = in.b, p0 = in.c;
      float ww = u + k;
      float pm = fmaxf(p0, ww);
      float e1 = expf(p0 - pm), e2 = expf(ww - pm);
      const float wkv = (e1 * a0 + e2 * v) / (e1 * b0 + e2);
      ex_store(p.rwkv + (size_t)b * C + c, r * wkv, tag);
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
      const float xin = ph.layer == 0 ? in.a
                                      : ex_finish(cx, in.wa, p.x + (size_t)b * C + c, phase_tag(p, pi - (p.version == 4 ? 2 : 3)));
      ex_store(p.xa + (size_t)b * C + c, xin + val[0], tag);
      break;
    }
    case PH_FFN_KR: {
      if (it < ph.split[0]) {
        const int f = it * ROWS + row;
        const float t = fmaxf(val[0], 0.f);
        ex_store(p.kk + (size_t)b * p.F + f, t * t, tag);
      } else {
        const int c = (it - ph.split[0]) * ROWS + row;
        ex_store(p.rr + (size_t)b * C + c, sigmoid_f(val[0]), tag);
      }
      break;
    }
    case PH_FFN_V: {
      const int c = it * ROWS + row;
      const float xin = ex_finish(cx, in.wa, p.xa + (size_t)b * C + c, phase_tag(p, pi - 2));
      const float rin = ex_finish(cx, in.wb, p.rr + (size_t)b * C + c, phase_tag(p, pi - 1));
      float xn = xin + rin * val[0];
      if (p.rescale_every > 0 && (ph.layer + 1) % p.rescale_every == 0) xn *= 0.5f;
      ex_store(p.x + (size_t)b * C + c, xn, tag);
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
      exch_t *dst = cls == 0 ? p.k5 : cls == 1 ? p.v5 : cls == 2 ? p.r5 : p.g5;
      float v = val[0];
      if (cls == 3) v = v * sigmoid_f(v);
      ex_store(dst + (size_t)b * C + c, v, tag);
      break;
    }
    default: break;
  }
}

// ---- all row blocks of a phase that belong to this CTA ----------------------------------------------
// One stream: the per-warp partial sums alternate between two buffers, so a row block needs one barrier (sums
// written -> sums read); the warps that run ahead write the other buffer, and the barrier of that next row block
// is what tells them the buffer after it is free again.  More streams: one buffer, a second barrier.
template <int FMT, int NB, int NT>
__device__ __forceinline__ void run_items(Ctx &cx, const PhaseDev &ph, int pi, int first) {
  constexpr int SB = n_streams<NB, NT>();
  constexpr int RN = red_n<NB, NT>();
  constexpr uint32_t RED_BUF = 3u * NW * RN * 4u;   // bytes of one partial-sum buffer
  const DecodeParams &p = *cx.p;
  const int KT = kt_max(FMT);
  const int nst = num_stages(FMT, ph.K);
  const uint32_t plane_b = (uint32_t)ph.K * NB * 2u;   // bytes per (vector, n-tile)
  const uint32_t vstride_b = plane_b * NT;
  const unsigned tag = phase_tag(p, pi);
  const int g = cx.lane >> 2, q = cx.lane & 3;
  // Phases with one matrix per row block (everything but the fused K,V,R of RWKV-4) take up to three row blocks per
  // barrier: their partial sums go to the three slots the fused phase uses for its three matrices, and thread
  // (slot, row, stream) runs the epilogue of row block `slot` of the batch.  The barrier, the cross-warp sum and the
  // epilogue's global stores are paid once per batch instead of once per 16 rows.
  constexpr int SLOT_THREADS = ROWS * SB;
  constexpr int MAX_GROUP = NCONS / SLOT_THREADS < 3 ? NCONS / SLOT_THREADS : 3;
  const int group = ph.n_sub == 1 ? MAX_GROUP : 1;
  const int eslot = cx.tid / SLOT_THREADS, etid = cx.tid - eslot * SLOT_THREADS;
  const int erow = etid / SB, eb = etid % SB;
  const bool prof = p.prof != nullptr && cx.tid == 0;
  const uint32_t xs_a = smem_u32(cx.sm.xs), ring_a = smem_u32(cx.sm.ring), red_a = smem_u32(cx.sm.red);
  const int last_kt = ph.K - (nst - 1) * KT;
  unsigned long long best = 0;   // head phase: packed arg-max over this thread's logits
  for (int it0 = first; it0 < ph.n_items; it0 += cx.G * group) {
    int n_in = 1;
    while (n_in < group && it0 + n_in * cx.G < ph.n_items) ++n_in;
    const int eit = it0 + eslot * cx.G;                       // row block this thread finishes
    const bool epi_thread = eslot < n_in && eb < p.B;
    EpiIn epi_in;
    if (epi_thread) epilogue_prefetch<FMT>(cx, ph, pi, eit, erow, eb, epi_in);
    const uint32_t red_it = red_a + (NB == 2 ? cx.red_buf * RED_BUF : 0u);
    const int n_mat = ph.n_sub == 1 ? n_in : ph.n_sub;        // matrices multiplied before the barrier
    for (int u = 0; u < n_mat; ++u) {
      const int it = ph.n_sub == 1 ? it0 + u * cx.G : it0;
      // which operand vector feeds this matrix
      int vec = ph.n_sub == 1 ? 0 : u;
      if (ph.kind == PH_FFN_KR) vec = it < ph.split[0] ? 0 : 1;
      else if (ph.kind == PH5_KVRG) vec = it / (p.C / ROWS);
      const uint32_t xv = xs_a + (uint32_t)vec * vstride_b;
      float acc[2][NT][4];
#pragma unroll
      for (int e = 0; e < 2; ++e)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[e][t][i] = 0.f;
      for (int s = 0; s < nst; ++s) {
        const int kt = s == nst - 1 ? last_kt : KT;
        if (!cx.ready) {
          const long long w0 = prof ? clock64() : 0;
          mbar_wait(&cx.sm.full[cx.slot], cx.parity, cx.sm.abort_flag, p.status, ST_TIMEOUT_FULL);
          if (prof) cx.wait_ns += clock64() - w0;
        }
        // look at the stage after this one now: the answer is back by the time this stage is multiplied
        const int cur = cx.slot;
        if (++cx.slot == p.n_stages) { cx.slot = 0; cx.parity ^= 1u; }
        cx.ready = mbar_test(&cx.sm.full[cx.slot], cx.parity);
        process_stage<FMT, NB, NT>(ring_a + (uint32_t)cur * cx.slot_b, kt / CHUNK_K, xv, plane_b, s * (KT / CHUNK_K),
                                   cx.warp, cx.lane, acc);
        __syncwarp();
        if (cx.lane == 0) mbar_arrive(&cx.sm.empty[cur]);
      }
      // this warp's share of the K split: hi + lo columns summed, parked in shared memory.
      // Accumulator c0,c1 = row g, columns 2q, 2q+1; c2,c3 = row g+8.
      const uint32_t r = red_it + (uint32_t)(u * NW + cx.warp) * (RN * 4u);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        float c0 = acc[0][t][0] + acc[1][t][0], c1 = acc[0][t][1] + acc[1][t][1];
        float c2 = acc[0][t][2] + acc[1][t][2], c3 = acc[0][t][3] + acc[1][t][3];
        if (NB == 2) {
          // columns 0 (hi) and 1 (lo) of the q == 0 lanes
          if (q == 0) { sts_f32(r + g * 4u, c0 + c1); sts_f32(r + (g + 8) * 4u, c2 + c3); }
        } else {
          // columns 0..3 = hi of streams 0..3 (lanes q = 0,1), columns 4..7 = lo (lanes q = 2,3)
          c0 += __shfl_xor_sync(0xffffffffu, c0, 2);
          c1 += __shfl_xor_sync(0xffffffffu, c1, 2);
          c2 += __shfl_xor_sync(0xffffffffu, c2, 2);
          c3 += __shfl_xor_sync(0xffffffffu, c3, 2);
          if (q < 2) {
            const int sb = t * 4 + 2 * q;
            sts_f32(r + (g * SB + sb) * 4u, c0); sts_f32(r + (g * SB + sb + 1) * 4u, c1);
            sts_f32(r + ((g + 8) * SB + sb) * 4u, c2); sts_f32(r + ((g + 8) * SB + sb + 1) * 4u, c3);
          }
        }
      }
    }
    bar_sync(BAR_CONS, NCONS);
    if (epi_thread) {
      float val[3] = {0.f, 0.f, 0.f};
#pragma unroll
      for (int u = 0; u < 3; ++u) {
        if (u < ph.n_sub) {
          const int slot = ph.n_sub == 1 ? eslot : u;
          float s = 0.f;
#pragma unroll
          for (int w = 0; w < NW; ++w) s += lds_f32(red_it + (uint32_t)((slot * NW + w) * RN + etid) * 4u);
          if (FMT == FMT_INT8) s *= epi_in.rscale[u];
          val[u] = s;
        }
      }
      epilogue(cx, ph, pi, tag, eit, erow, eb, val, epi_in);
      if (ph.kind == PH_HEAD && p.amax && eit * ROWS + erow < p.V) {
        unsigned u = __float_as_uint(val[0]);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        const unsigned long long w = ((unsigned long long)u << 32) | (0xffffffffu - (unsigned)(eit * ROWS + erow));
        best = w > best ? w : best;
      }
    }
    if (NB == 2) cx.red_buf ^= 1u;
    else bar_sync(BAR_CONS, NCONS);   // the partial sums are read: the next row block may overwrite them
  }
  // (the head phase has one matrix per row block: every thread with eslot < 3 may hold a candidate)
  if (ph.kind == PH_HEAD && p.amax && eslot < MAX_GROUP && eb < p.B && best) atomicMax(p.amax + eb, best);
}

// ---- v5 state update + readout: units of (stream, head, 16 value columns) ----------------------------
__device__ __forceinline__ void phase_wkv5(Ctx &cx, const PhaseDev &ph, int pi) {
  const DecodeParams &p = *cx.p;
  const int C = p.C, H = p.H;
  const int units = p.B * H * 4;
  const unsigned in_tag = phase_tag(p, pi - 1), tag = phase_tag(p, pi);
  float *scratch = reinterpret_cast<float *>(cx.sm.xs);  // [NW][16] partial readouts
  const int first = (cx.cta + cx.G - ph.rot) % cx.G;
  for (int un = first; un < units; un += cx.G) {
    const int b = un / (H * 4), h = (un / 4) % H, j0 = (un & 3) * 16;
    const int i = cx.tid >> 2, jq = (cx.tid & 3) * 4;
    uint8_t *stb = p.state + (size_t)b * p.state_stride + (size_t)ph.layer * p.layer_stride;
    float *S = reinterpret_cast<float *>(stb + off_mid(C, p.act_fp16)) + (size_t)h * 4096;
    float4 *sp = reinterpret_cast<float4 *>(S + i * 64 + j0 + jq);
    float4 s = *sp;
    // k, r and v are requested together (a wait that checks its answer before the next request goes out costs a
    // round trip to L2 each); whatever has not arrived is waited for afterwards
    const exch_t *kp = p.k5 + (size_t)b * C + h * 64 + i, *rp = p.r5 + (size_t)b * C + h * 64 + i;
    const exch_t *vp = p.v5 + (size_t)b * C + h * 64 + j0 + jq;
    const exch_t kw = ex_load_raw(kp), rw = ex_load_raw(rp);
    const uint4 vw = ex_load_raw4(vp);
    const float ki = ex_ready(kw, in_tag) ? ex_value(kw) : ex_wait1(cx, kp, in_tag);
    const float ri = ex_ready(rw, in_tag) ? ex_value(rw) : ex_wait1(cx, rp, in_tag);
    float4 vj;
    if (!ex_decode4(vw, in_tag, vj)) vj = ex_wait4(cx, vp, in_tag);
    const float u = p.version == 50 ? __ldg(ph.aux0 + h) : __ldg(ph.aux0 + h * 64 + i);
    const float w = p.version == 50 ? __ldg(ph.aux1 + h) : __ldg(ph.aux1 + h * 64 + i);
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
      ex_store(p.o5 + (size_t)b * C + h * 64 + j0 + cx.tid, t, tag);
    }
    bar_sync(BAR_CONS, NCONS);
  }
}

// ------------------------------------------------------------------------------------------------
template <int FMT, int NB, int NT>
__device__ __forceinline__ void consumer(Ctx &cx) {
  const DecodeParams &p = *cx.p;
  const bool prof = p.prof != nullptr && cx.tid == 0;
  // the next phase's descriptor is requested a phase ahead: its load latency is off the hand-over path
  PhaseDev nxt = p.phases[0];
  for (int pi = 0; pi < p.n_phases; ++pi) {
    cx.pc[0] = prof ? clock64() : 0;  // trace
    const PhaseDev ph = nxt;
    if (pi + 1 < p.n_phases) nxt = p.phases[pi + 1];
    const int first = (cx.cta + cx.G - ph.rot) % cx.G;
    if (ph.kind == PH5_WKV) {
      if (first < p.B * p.H * 4) phase_wkv5(cx, ph, pi);
      continue;
    }
    if (first >= ph.n_items) continue;   // no row block here: nothing to read, nothing to write
    cx.prof_phase = pi;
    if (prof) p.prof[((size_t)cx.cta * p.n_phases + pi) * 8 + 0] = globaltimer_ns();
    cx.pc[1] = cx.pc[2] = cx.pc[3] = cx.pc[4] = prof ? clock64() : 0;  // trace
    if (is_ln_phase(ph.kind)) {
      prologue_ln<NB, NT>(cx, ph, pi, phase_tag(p, pi - 1));
    } else if (ph.kind == PH_ATT_O) {
      if (p.version == 4) prologue_vec<NB, NT>(cx, p.rwkv, p.C, phase_tag(p, pi - 1));
      else prologue_gn_gate<NB, NT>(cx, ph, phase_tag(p, pi - 1), phase_tag(p, pi - 2));
    } else if (ph.kind == PH_FFN_V) {
      prologue_vec<NB, NT>(cx, p.kk, p.F, phase_tag(p, pi - 1));
    } else if (ph.kind == PH_MATVEC) {
      prologue_plain<NB, NT>(cx, reinterpret_cast<const float *>(p.kk), ph.K);
    }
    if (prof) { unsigned long long *pr = p.prof + ((size_t)cx.cta * p.n_phases + pi) * 8; pr[4] = cx.pc[1] - cx.pc[0]; pr[5] = cx.pc[2] - cx.pc[1]; pr[6] = cx.pc[3] - cx.pc[2]; pr[7] = cx.pc[4] - cx.pc[3]; }  // trace
    if (prof) { p.prof[((size_t)cx.cta * p.n_phases + pi) * 8 + 1] = globaltimer_ns(); cx.wait_ns = 0; }
    run_items<FMT, NB, NT>(cx, ph, pi, first);
    if (prof) { p.prof[((size_t)cx.cta * p.n_phases + pi) * 8 + 2] = globaltimer_ns(); p.prof[((size_t)cx.cta * p.n_phases + pi) * 8 + 3] = cx.wait_ns; }
  }
}

// Walks this CTA's weight tiles in the order the consumers use them: phases in order, the CTA's row
// blocks of the phase, the matrices fused in a row block, the stages of a matrix.
template <int FMT>
struct TileIter {
  const DecodeParams *p;
  int cta, G;
  int pi, it, u, s, nst;
  PhaseDev ph;
  const uint8_t *src;
  bool done;

  __device__ __forceinline__ void load_phase() {
    // advance pi to the next phase in which this CTA owns a row block
    while (pi < p->n_phases) {
      ph = p->phases[pi];
      if (ph.n_items > 0) {
        it = (cta + G - ph.rot) % G;
        if (it < ph.n_items) {
          nst = num_stages(FMT, ph.K);
          u = 0; s = 0;
          src = ph.w + (size_t)it * rowblock_bytes(FMT, ph.K) * ph.n_sub;
          return;
        }
      }
      ++pi;
    }
    done = true;
  }
  __device__ __forceinline__ void init(const DecodeParams *pp, int cta_, int G_) {
    p = pp; cta = cta_; G = G_; pi = 0; done = false;
    load_phase();
  }
  __device__ __forceinline__ uint32_t bytes() const {
    const int KT = kt_max(FMT);
    return stage_bytes(FMT, min(KT, ph.K - s * KT));
  }
  __device__ __forceinline__ void next() {
    src += bytes();
    if (++s < nst) return;
    s = 0;
    if (++u < ph.n_sub) return;
    u = 0;
    it += G;
    if (it < ph.n_items) {
      src = ph.w + (size_t)it * rowblock_bytes(FMT, ph.K) * ph.n_sub;
      return;
    }
    ++pi;
    load_phase();
  }
};

__device__ __forceinline__ void prefetch_l2(const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// One thread per CTA.  Keeps the shared-memory ring full; optionally asks L2 for tiles further ahead.
template <int FMT>
__device__ __forceinline__ void producer(Ctx &cx) {
  const DecodeParams &p = *cx.p;
  TileIter<FMT> ld, pf;
  ld.init(&p, cx.cta, cx.G);
  pf.init(&p, cx.cta, cx.G);
  long long ld_bytes = 0, pf_bytes = 0;
  const long long window = (long long)p.l2_prefetch_bytes;
  int slot = 0;
  uint32_t parity = 1;  // a fresh barrier reads as "previous phase complete"
  uint32_t par_parity = 1;
  int par_pi = -1;      // phase whose LayerNorm parameters were staged last
  bool live = true;
  const uint64_t pol = l2_evict_first_policy();
  while (!ld.done) {
    while (window > 0 && !pf.done && pf_bytes - ld_bytes < window) {
      const uint32_t b = pf.bytes();
      if (pf_bytes >= ld_bytes + (long long)p.n_stages * cx.slot_b) prefetch_l2(pf.src, b);  // beyond the ring
      pf_bytes += b;
      pf.next();
    }
    if (cx.sm.par && ld.pi != par_pi && is_ln_phase(ld.ph.kind)) {
      // first tile of a LayerNorm phase: its parameters go in first, once the consumers have left the previous set
      if (!mbar_wait(cx.sm.par_free, par_parity, cx.sm.abort_flag, p.status, ST_TIMEOUT_EMPTY)) { live = false; break; }
      par_parity ^= 1u;
      ln_stage_params(cx, ln_args(p, ld.ph));
      par_pi = ld.pi;
    }
    const uint32_t bytes = ld.bytes();
    if (!mbar_wait(&cx.sm.empty[slot], parity, cx.sm.abort_flag, p.status, ST_TIMEOUT_EMPTY)) {
      live = false;
      break;
    }
    mbar_expect_tx(&cx.sm.full[slot], bytes);
    bulk_g2s_hint(cx.sm.ring + (size_t)slot * cx.slot_b, ld.src, bytes, &cx.sm.full[slot], pol);
    ld_bytes += bytes;
    ld.next();
    if (++slot == p.n_stages) { slot = 0; parity ^= 1u; }
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
  cx.slot = 0; cx.parity = 0; cx.wait_ns = 0; cx.prof_phase = 0; cx.red_buf = 0; cx.ready = false;
  cx.slot_b = slot_bytes(FMT);
  size_t o_red, o_par, o_xs, o_ring;
  smem_layout<NB, NT>(FMT, p.C, p.F, p.version, p.n_stages, p.vecs16 != nullptr, &o_red, &o_par, &o_xs, &o_ring);
  cx.sm.par = par_bytes<NB, NT>(p.C, p.vecs16 != nullptr) ? reinterpret_cast<float *>(smem + o_par) : nullptr;
  cx.par_parity = 0;
  cx.sm.par_bar = reinterpret_cast<uint64_t *>(smem + 200);
  cx.sm.par_free = reinterpret_cast<uint64_t *>(smem + 208);
  cx.sm.full = reinterpret_cast<uint64_t *>(smem);
  cx.sm.empty = cx.sm.full + MAX_STAGES;
  cx.sm.abort_flag = reinterpret_cast<volatile int *>(smem + 256);
  cx.sm.ln_red = reinterpret_cast<float *>(smem + 320);
  cx.sm.red = reinterpret_cast<float *>(smem + o_red);
  cx.sm.xs = reinterpret_cast<__half *>(smem + o_xs);
  cx.sm.ring = smem + o_ring;

  if (cx.tid == 0) {
    for (int s = 0; s < p.n_stages; ++s) {
      mbar_init(&cx.sm.full[s], 1);
      mbar_init(&cx.sm.empty[s], NW);
    }
    *cx.sm.abort_flag = 0;
    mbar_init(cx.sm.par_bar, 1);
    mbar_init(cx.sm.par_free, NW);
    mbar_fence_init();
  }
  __syncthreads();

  // Register hand-over between the warp groups (the launch gives every thread 168): the producer group
  // keeps 40 and the two consumer groups grow to 232, enough to hold a row block's accumulators, the
  // prefetched epilogue inputs and a LayerNorm prologue's parameters without touching local memory.
  if (cx.warp >= NW) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (cx.warp == NW && cx.lane == 0) producer<FMT>(cx);
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    consumer<FMT, NB, NT>(cx);
  }
}

__global__ void unpack_ids_kernel(const unsigned long long *packed, int n, int32_t *out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (int32_t)(0xffffffffu - (unsigned)packed[i]);
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
size_t decode_smem_bytes(int fmt, int mode, int C, int F, int version, int n_stages, int par16) {
  size_t a, b, c, d;
  switch (mode) {
    case 0: return smem_layout<2, 1>(fmt, C, F, version, n_stages, par16, &a, &b, &c, &d);
    case 1: return smem_layout<8, 1>(fmt, C, F, version, n_stages, par16, &a, &b, &c, &d);
    default: return smem_layout<8, 2>(fmt, C, F, version, n_stages, par16, &a, &b, &c, &d);
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

namespace {
// One thread waits on an mbarrier that nobody ever arrives at, through the same bounded-wait helper every kernel
// here uses, with the given limit: the wait must give up, record ST_TIMEOUT_FULL and let the kernel end normally.
__global__ void wait_selftest_kernel(int *status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag, status, ST_TIMEOUT_FULL, limit_ns);
}
}  // namespace

cudaError_t launch_wait_selftest(int *status, unsigned long long limit_ns, cudaStream_t st) {
  wait_selftest_kernel<<<1, 32, 0, st>>>(status, limit_ns);
  return cudaGetLastError();
}

cudaError_t launch_unpack_ids(const unsigned long long *packed, int n, int32_t *out, cudaStream_t st) {
  unpack_ids_kernel<<<(n + 255) / 256, 256, 0, st>>>(packed, n, out);
  return cudaGetLastError();
}

}  // namespace frb
