// Seq mode (prompt processing): T tokens of one stream at once.
//
// Replaces the reference's seq path for RWKV-5.x: def::ModelForwardSeq (kernels/default/model_forward_seq.cpp:48-184),
// _ATT_SEQ_V5_2 + rwkv5_2_kernel_forward (kernels/cuda/att_seq.cu:258-322, 368-423) and _FFN_SEQ
// (kernels/cuda/ffn_seq.cu:65-87).  The projections are [T, K] x [K, N] GEMMs on the tcgen05 tensor cores
// (operands staged by TMA, accumulator in TMEM, epilogue fused); LayerNorm + token shift, the per-head state scan
// and GroupNorm + gate are bandwidth-bound row kernels around them.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <utility>

#include "common.cuh"
#include "internal.h"

namespace frb {

// SMs of the current device (asked once per device): grids and split-K factors are sized from it
int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

// Every kernel of the seq / batch chain goes through here.  With FR_B200_PDL != 0 (the default) the launch carries
// the programmatic stream-serialisation attribute: the kernel's CTAs may be scheduled, and run their set-up, while the
// kernel before it in the stream drains; each kernel calls pdl_wait() before it touches global memory, so the data
// dependences are those of plain stream order.
bool pdl_enabled() {
  static const int on = [] { const char *v = getenv("FR_B200_PDL"); return !(v && v[0] == '0'); }();
  return on != 0;
}
template <typename... KArgs, typename... Args>
cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// ------------------------------------------------------------------------------------------------
// tcgen05 GEMM: out[M, N] = epilogue((A + A2)[M, K] . (Bt + Bt2)[N, K]^T), fp16 operands (both K-major), fp32
// accumulate.  A2 (optional) holds what rounding the activations to fp16 lost: its tiles travel in the same ring slot
// and multiply the same B tile.  Bt2 (optional, int4 weights) is a second pass over K.
// One CTA per 128 x 256 output tile; K is walked in 64-wide slices through a 4-deep TMA ring.
//   warp 0 (one lane): TMA producer          warp 1 (one lane): MMA issue; the warp owns the TMEM allocation
//   warps 2..5: epilogue, one TMEM lane quadrant (32 rows) each
constexpr int GBM = 128, GBK = 64;
constexpr int G_THREADS = 192;
constexpr uint32_t G_A_BYTES = GBM * GBK * 2;
constexpr int ST_GEMM_TIMEOUT = 201;

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
// shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 halfs), 128-byte swizzle, eight-row
// groups 1024 bytes apart: start address / 16 in bits 0-13, leading offset (unused for swizzled K-major) = 1 in
// bits 16-29, stride offset 1024 / 16 in bits 32-45, descriptor version 1 in bits 46-47, layout 2 (128B) in bits 61-63
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor, kind::f16: D = f32 (bits 4-5 = 1), A = B = f16 (0), both K-major (0), N / 8 in bits 17-22,
// M / 16 in bits 24-28
// (built per tile width inside the kernel)

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// the tensor maps are launch parameters: their first use would be a cold fetch in front of the first tile
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// the result is rounded to fp16: the fast exponential and division are exact enough
__device__ __forceinline__ float sigmoid_g(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }

// Epilogue of 32 consecutive columns of one output row (16-byte accesses when all 32 columns exist).
__device__ __forceinline__ float epi_half_op(int epi, float a) {
  if (epi == GEMM_EPI_SILU_F16) return a * sigmoid_g(a);
  if (epi == GEMM_EPI_SIGMOID_F16) return sigmoid_g(a);
  if (epi == GEMM_EPI_RELU2_F16) { a = fmaxf(a, 0.f); return a * a; }
  return a;
}
__device__ __forceinline__ void gemm_epilogue_row(const GemmArgs &g, int row, int col0, const uint32_t (&acc)[32]) {
  const int ncol = min(32, g.N - col0);
  if (ncol <= 0) return;
  const size_t o = (size_t)row * g.ldo + col0;
  const bool full = ncol == 32 && (g.ldo & 7) == 0;
  if (g.epi == GEMM_EPI_F32) {
    float *out = reinterpret_cast<float *>(g.out) + o;
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4 *>(out + i) = make_float4(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]),
                                                           __uint_as_float(acc[i + 2]), __uint_as_float(acc[i + 3]));
    } else {
      for (int i = 0; i < ncol; ++i) out[i] = __uint_as_float(acc[i]);
    }
    return;
  }
  if (g.epi == GEMM_EPI_ADD_F32 || g.epi == GEMM_EPI_MULADD_F32) {
    // residual stream (fp32): x + acc, or x + r * acc (r fp16), optionally scaled
    float *out = reinterpret_cast<float *>(g.out) + o;
    const float *x = reinterpret_cast<const float *>(g.aux0) + o;
    const __half *r = reinterpret_cast<const __half *>(g.aux1) + o;
    const bool mul = g.epi == GEMM_EPI_MULADD_F32;
    if (mul && g.aux1_lo) {
      const __half *rl = reinterpret_cast<const __half *>(g.aux1_lo) + o;
      for (int i = 0; i < ncol; ++i)
        out[i] = (x[i] + (__half2float(r[i]) + __half2float(rl[i])) * __uint_as_float(acc[i])) * g.scale;
      return;
    }
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        const float4 x0 = *reinterpret_cast<const float4 *>(x + i), x1 = *reinterpret_cast<const float4 *>(x + i + 4);
        float rr[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
        if (mul) {
          const uint4 rw = *reinterpret_cast<const uint4 *>(r + i);
          const float2 r0 = __half22float2(*reinterpret_cast<const __half2 *>(&rw.x)), r1 = __half22float2(*reinterpret_cast<const __half2 *>(&rw.y));
          const float2 r2 = __half22float2(*reinterpret_cast<const __half2 *>(&rw.z)), r3 = __half22float2(*reinterpret_cast<const __half2 *>(&rw.w));
          rr[0] = r0.x; rr[1] = r0.y; rr[2] = r1.x; rr[3] = r1.y; rr[4] = r2.x; rr[5] = r2.y; rr[6] = r3.x; rr[7] = r3.y;
        }
        float4 y0, y1;
        y0.x = (x0.x + rr[0] * __uint_as_float(acc[i])) * g.scale;     y0.y = (x0.y + rr[1] * __uint_as_float(acc[i + 1])) * g.scale;
        y0.z = (x0.z + rr[2] * __uint_as_float(acc[i + 2])) * g.scale; y0.w = (x0.w + rr[3] * __uint_as_float(acc[i + 3])) * g.scale;
        y1.x = (x1.x + rr[4] * __uint_as_float(acc[i + 4])) * g.scale; y1.y = (x1.y + rr[5] * __uint_as_float(acc[i + 5])) * g.scale;
        y1.z = (x1.z + rr[6] * __uint_as_float(acc[i + 6])) * g.scale; y1.w = (x1.w + rr[7] * __uint_as_float(acc[i + 7])) * g.scale;
        *reinterpret_cast<float4 *>(out + i) = y0;
        *reinterpret_cast<float4 *>(out + i + 4) = y1;
      }
    } else {
      for (int i = 0; i < ncol; ++i) {
        float a = __uint_as_float(acc[i]);
        if (mul) a *= __half2float(r[i]);
        out[i] = (x[i] + a) * g.scale;
      }
    }
    return;
  }
  __half *out = reinterpret_cast<__half *>(g.out) + o;
  if (g.out_lo) {
    // the consumer of this output wants it as a hi + lo pair (batched decode keeps ~22 bits between projections)
    __half *lo = reinterpret_cast<__half *>(g.out_lo) + o;
    for (int i = 0; i < ncol; ++i) {
      const float v = epi_half_op(g.epi, __uint_as_float(acc[i]));
      const __half h = __float2half_rn(v);
      out[i] = h;
      lo[i] = __float2half_rn(v - __half2float(h));
    }
    return;
  }
  if (full) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint4 w;
      __half2 h;
      h = __floats2half2_rn(epi_half_op(g.epi, __uint_as_float(acc[i])), epi_half_op(g.epi, __uint_as_float(acc[i + 1])));     w.x = *reinterpret_cast<uint32_t *>(&h);
      h = __floats2half2_rn(epi_half_op(g.epi, __uint_as_float(acc[i + 2])), epi_half_op(g.epi, __uint_as_float(acc[i + 3]))); w.y = *reinterpret_cast<uint32_t *>(&h);
      h = __floats2half2_rn(epi_half_op(g.epi, __uint_as_float(acc[i + 4])), epi_half_op(g.epi, __uint_as_float(acc[i + 5]))); w.z = *reinterpret_cast<uint32_t *>(&h);
      h = __floats2half2_rn(epi_half_op(g.epi, __uint_as_float(acc[i + 6])), epi_half_op(g.epi, __uint_as_float(acc[i + 7]))); w.w = *reinterpret_cast<uint32_t *>(&h);
      *reinterpret_cast<uint4 *>(out + i) = w;
    }
  } else {
    for (int i = 0; i < ncol; ++i) out[i] = __float2half_rn(epi_half_op(g.epi, __uint_as_float(acc[i])));
  }
}

// Up to four GEMMs with the same M in one launch (grid.x walks their N tiles back to back, heaviest first): the
// attention projections of a layer, or the two channel-mix projections that read the LayerNorm output.
struct GemmGroup {
  int n;
  int stages;                           // ring depth (2..4); packed-weight GEMM: weight slots
  int estages;                          // packed-weight GEMM: buffers (expanded weights + X; stage_bytes = the X part)
  uint32_t wbox;                        // packed-weight GEMM: bytes per row of a weight slot (64 or 128)
  uint32_t stage_bytes;                 // bytes per ring slot: [A hi tiles][A lo tiles, if any problem has them][B tile]
  int split;                            // split-K factor (grid.z); > 1: CTAs write raw partial sums to GemmArgs::raw
  int dual;                             // 1: the slot has room for the low halves of A (128-row tiles);
                                        // 0: low halves of A, if any, are a further pass over K (256-row tiles: a
                                        //    slot with both would leave a 2-deep ring)
  int tile_start[GEMM_GROUP_MAX + 1];   // first grid.x index of each problem
  GemmArgs p[GEMM_GROUP_MAX];
};
struct alignas(64) GemmMaps {
  CUtensorMap a[GEMM_GROUP_MAX], a2[GEMM_GROUP_MAX], b[GEMM_GROUP_MAX], b2[GEMM_GROUP_MAX];
};

// MT = 128-row sub-tiles per CTA (1: 128 x BN output tile; 2: 256 x BN, two accumulators sharing every B tile --
// half again as many flops per byte fetched from L2).  BN = 256 for prompts; BN = 64 with split-K (grid.z) when
// there are only a few hundred rows (batched decode): the step is bound by streaming the weights, so the number of
// CTAs that each stream a distinct slice is what counts; the partial sums go to per-split slabs that
// gemm_finish_kernel adds up in a fixed order before the epilogue.
template <int MT, int BN>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_f16_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ GemmGroup grp) {
  constexpr int GBN = BN;
  constexpr uint32_t G_B_BYTES = BN * GBK * 2;
  constexpr uint32_t G_IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GBM >> 4) << 24);
  const int STAGES = grp.stages;
  const uint32_t STAGE_BYTES = grp.stage_bytes;
  const uint32_t B_OFF = (uint32_t)(grp.dual ? 2 : 1) * MT * G_A_BYTES;   // the B tile follows the A tiles
  constexpr uint32_t TMEM_COLS = MT * GBN < 32 ? 32 : MT * GBN;
  extern __shared__ uint8_t gsm_raw[];
  // barriers in the first KB, tiles from the next 1024-byte boundary
  uint8_t *gsm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *full = reinterpret_cast<uint64_t *>(gsm);
  uint64_t *empty = full + 4;
  uint64_t *acc_full = empty + 4;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t tiles = smem_u32(gsm + 1024);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pi = 0;
  while (pi + 1 < grp.n && (int)blockIdx.x >= grp.tile_start[pi + 1]) ++pi;
  const GemmArgs &g = grp.p[pi];
  const int tile_m = blockIdx.y, tile_n = blockIdx.x - grp.tile_start[pi];
  const int num_k1 = g.K / GBK;
  // the low halves of A (A2) ride in the same ring slot as the high halves and meet the same B tile; the low
  // halves of B (Bt2) are a second pass over K into the same accumulator
  const bool has_lo = g.A2 != nullptr && grp.dual, lo_pass = g.A2 != nullptr && !grp.dual;
  // split-K: this CTA covers K slices [kz0, kz0 + nkz) of every pass
  const int kz0 = (int)((long long)blockIdx.z * num_k1 / grp.split), nkz = (int)((long long)(blockIdx.z + 1) * num_k1 / grp.split) - kz0;
  const int num_k = nkz * (1 + (lo_pass ? 1 : 0) + (g.Bt2 ? 1 : 0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  pdl_wait();   // operands and epilogue inputs come from the kernels before this one

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % STAGES;
        const uint32_t parity = ((kb / STAGES) & 1) ^ 1;   // a fresh barrier reads as "previous phase complete"
        if (!mbar_wait(&empty[s], parity, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
        const int pass = kb / nkz, kk = kz0 + kb - pass * nkz;
        const bool lo_now = has_lo && pass == 0;   // the (lo A) x (lo B) term is below fp32 resolution: skipped
        const bool a_is_lo = lo_pass && pass == 1, b_is_lo = pass > 0 && !a_is_lo;
        mbar_expect_tx(&full[s], (uint32_t)(lo_now ? 2 : 1) * MT * G_A_BYTES + G_B_BYTES);
        const uint32_t a_dst = tiles + (uint32_t)s * STAGE_BYTES;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          tma_load_2d(a_dst + (uint32_t)mt * G_A_BYTES, a_is_lo ? &maps.a2[pi] : &maps.a[pi], kk * GBK, (tile_m * MT + mt) * GBM, &full[s]);
          if (lo_now) tma_load_2d(a_dst + (uint32_t)(MT + mt) * G_A_BYTES, &maps.a2[pi], kk * GBK, (tile_m * MT + mt) * GBM, &full[s]);
        }
        tma_load_2d(a_dst + B_OFF, b_is_lo ? &maps.b2[pi] : &maps.b[pi], kk * GBK, tile_n * GBN, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(&full[s], (kb / STAGES) & 1, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
        tc_fence_after();
        const uint32_t a_addr = tiles + (uint32_t)s * STAGE_BYTES;
        const uint64_t bd = umma_desc_k128(a_addr + B_OFF);
        const bool lo_now = has_lo && kb < nkz;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t ad = umma_desc_k128(a_addr + (uint32_t)mt * G_A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < GBK / 16; ++k4)   // 16 inputs = 32 bytes further along the swizzled rows
            umma_f16(tmem_base + (uint32_t)mt * GBN, ad + (uint64_t)(k4 * 2), bd + (uint64_t)(k4 * 2), G_IDESC, (kb | k4) != 0);
          if (lo_now) {
            const uint64_t al = umma_desc_k128(a_addr + (uint32_t)(MT + mt) * G_A_BYTES);
#pragma unroll
            for (int k4 = 0; k4 < GBK / 16; ++k4)
              umma_f16(tmem_base + (uint32_t)mt * GBN, al + (uint64_t)(k4 * 2), bd + (uint64_t)(k4 * 2), G_IDESC, 1u);
          }
        }
        umma_commit(&empty[s]);   // the slot is free once these MMAs have read it
      }
      umma_commit(acc_full);      // the accumulators are complete once every MMA has retired
    }
  } else {
    // epilogue warps 2..5 -> TMEM lane quadrants 2, 3, 0, 1
    const int quad = warp & 3;
    const bool ok = mbar_wait(acc_full, 0, abort_flag, g.status, ST_GEMM_TIMEOUT);
    tc_fence_after();
    if (ok) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int row = (tile_m * MT + mt) * GBM + quad * 32 + lane;
        if ((tile_m * MT + mt) * GBM >= g.M) break;   // warp-uniform
        for (int c0 = 0; c0 < GBN; c0 += 32) {
          if (tile_n * GBN + c0 >= g.N) break;   // warp-uniform
          uint32_t acc[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(mt * GBN + c0), acc);
          if (grp.split > 1) {
            // raw partial sums of this K range: slab blockIdx.z of [split][M][N]
            if (row < g.M) {
              float *dst = g.raw + ((size_t)blockIdx.z * g.M + row) * g.N + tile_n * GBN + c0;
              const int ncol = min(32, g.N - (tile_n * GBN + c0));
              if (ncol == 32 && (g.N & 3) == 0) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                  *reinterpret_cast<float4 *>(dst + i) = make_float4(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]),
                                                                     __uint_as_float(acc[i + 2]), __uint_as_float(acc[i + 3]));
              } else {
                for (int i = 0; i < ncol; ++i) dst[i] = __uint_as_float(acc[i]);
              }
            }
            continue;
          }
          if (g.col_scale) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = tile_n * GBN + c0 + i;
              acc[i] = __float_as_uint(__uint_as_float(acc[i]) * (col < g.N ? __half2float(g.col_scale[col]) : 0.f));
            }
          }
          if (row < g.M) gemm_epilogue_row(g, row, tile_n * GBN + c0, acc);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Few rows (batched decode: one row per stream, or a short prompt): the same product with the operands' roles
// swapped, out^T[N, M] = W^T[N, K] . X[M, K]^T.  The 128 MMA rows are 128 output channels of the weight matrix, the
// MMA columns are the BN rows of X (32 .. 256), so a ring slot is 16 KB of weights plus a small X tile instead of a
// 128-row X tile that is mostly zero fill plus 8 KB of weights: several times the weight bytes in flight per SM,
// which is what a step that streams every weight once is bound by.  The low halves of X (A2) and of the weights
// (Bt2) sit in the same slot and multiply into the same accumulator; (lo W) x (lo X) is below fp32 resolution.
// The accumulator holds out^T: TMEM lane = output channel, column = row of X; the epilogue warps write with the
// lanes along the channels (coalesced), either the finished values or the split-K slabs gemm_finish_kernel sums.
constexpr int WT_MAX_STAGES = 8;

__device__ __forceinline__ void epi_store_one(const GemmArgs &g, int row, int col, float a) {
  const size_t o = (size_t)row * g.ldo + col;
  if (g.epi == GEMM_EPI_F32) {
    reinterpret_cast<float *>(g.out)[o] = a;
  } else if (g.epi == GEMM_EPI_ADD_F32) {
    reinterpret_cast<float *>(g.out)[o] = (reinterpret_cast<const float *>(g.aux0)[o] + a) * g.scale;
  } else if (g.epi == GEMM_EPI_MULADD_F32) {
    float r = __half2float(reinterpret_cast<const __half *>(g.aux1)[o]);
    if (g.aux1_lo) r += __half2float(reinterpret_cast<const __half *>(g.aux1_lo)[o]);
    reinterpret_cast<float *>(g.out)[o] = (reinterpret_cast<const float *>(g.aux0)[o] + r * a) * g.scale;
  } else {
    const float e = epi_half_op(g.epi, a);
    const __half h = __float2half_rn(e);
    reinterpret_cast<__half *>(g.out)[o] = h;
    if (g.out_lo) reinterpret_cast<__half *>(g.out_lo)[o] = __float2half_rn(e - __half2float(h));
  }
}

// grp.dual here: bit 0 = some problem has A2 (slot holds an X lo tile), bit 1 = some problem has Bt2 (W lo tile)
template <int BN>
__global__ void __launch_bounds__(G_THREADS, 2)
gemm_wt_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ GemmGroup grp) {
  constexpr uint32_t X_BYTES = BN * GBK * 2;
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GBM >> 4) << 24);
  // up to 128 rows the hi and lo tiles of X, back to back in the slot, are one B operand of 2 BN rows (accumulator
  // columns [0, BN) and [BN, 2 BN), added up by the epilogue): an MMA with few columns costs about as much as a wide one
  constexpr bool FUSE_LO = BN <= 128;
  constexpr uint32_t IDESC2 = (1u << 4) | ((uint32_t)((2 * BN) >> 3) << 17) | ((uint32_t)(GBM >> 4) << 24);
  constexpr uint32_t TMEM_COLS = FUSE_LO ? 2 * BN : BN;
  const int STAGES = grp.stages;
  const uint32_t STAGE_BYTES = grp.stage_bytes;
  const uint32_t X_OFF = ((grp.dual & 2) ? 2u : 1u) * G_A_BYTES, XLO_OFF = X_OFF + X_BYTES;
  extern __shared__ uint8_t gsm_raw[];
  uint8_t *gsm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *full = reinterpret_cast<uint64_t *>(gsm);
  uint64_t *empty = full + WT_MAX_STAGES;
  uint64_t *acc_full = empty + WT_MAX_STAGES;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t tiles = smem_u32(gsm + 1024);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pi = 0;
  while (pi + 1 < grp.n && (int)blockIdx.x >= grp.tile_start[pi + 1]) ++pi;
  const GemmArgs &g = grp.p[pi];
  const int tile_n = blockIdx.x - grp.tile_start[pi], m0 = blockIdx.y * BN;
  const int num_k1 = g.K / GBK;
  const int kz0 = (int)((long long)blockIdx.z * num_k1 / grp.split), nkz = (int)((long long)(blockIdx.z + 1) * num_k1 / grp.split) - kz0;
  const bool x_lo = g.A2 != nullptr, w_lo = g.Bt2 != nullptr;

  if (threadIdx.x == 64) {
    prefetch_tmap(&maps.b[pi]); prefetch_tmap(&maps.a[pi]);
    if (x_lo) prefetch_tmap(&maps.a2[pi]);
    if (w_lo) prefetch_tmap(&maps.b2[pi]);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  // The weights are constants: the ring's first round of weight tiles is on its way before the kernels ahead of this
  // one have finished.  What they wrote (X, the epilogue's inputs and outputs) is touched only after pdl_wait(): by
  // the X loads and by the epilogue warps.

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t w_bytes = (w_lo ? 2u : 1u) * G_A_BYTES, x_bytes = (x_lo ? 2u : 1u) * X_BYTES;
      const int pre = nkz < STAGES ? nkz : STAGES;
      for (int kb = 0; kb < pre; ++kb) {
        mbar_expect_tx_only(&full[kb], w_bytes);
        const uint32_t dst = tiles + (uint32_t)kb * STAGE_BYTES;
        tma_load_2d(dst, &maps.b[pi], (kz0 + kb) * GBK, tile_n * GBM, &full[kb]);
        if (w_lo) tma_load_2d(dst + G_A_BYTES, &maps.b2[pi], (kz0 + kb) * GBK, tile_n * GBM, &full[kb]);
      }
      pdl_wait();
      for (int kb = 0; kb < nkz; ++kb) {
        const int s = kb % STAGES;
        const uint32_t dst = tiles + (uint32_t)s * STAGE_BYTES;
        const int kx = (kz0 + kb) * GBK;
        if (kb >= pre) {
          if (!mbar_wait(&empty[s], ((kb / STAGES) & 1) ^ 1, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
          mbar_expect_tx(&full[s], w_bytes + x_bytes);
          tma_load_2d(dst, &maps.b[pi], kx, tile_n * GBM, &full[s]);
          if (w_lo) tma_load_2d(dst + G_A_BYTES, &maps.b2[pi], kx, tile_n * GBM, &full[s]);
        } else {
          mbar_expect_tx(&full[s], x_bytes);
        }
        tma_load_2d(dst + X_OFF, &maps.a[pi], kx, m0, &full[s]);
        if (x_lo) tma_load_2d(dst + XLO_OFF, &maps.a2[pi], kx, m0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < nkz; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(&full[s], (kb / STAGES) & 1, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
        tc_fence_after();
        const uint32_t base = tiles + (uint32_t)s * STAGE_BYTES;
        const uint64_t wd = umma_desc_k128(base), xd = umma_desc_k128(base + X_OFF);
        const bool wide = FUSE_LO && x_lo;
#pragma unroll
        for (int k4 = 0; k4 < GBK / 16; ++k4)
          umma_f16(tmem_base, wd + (uint64_t)(k4 * 2), xd + (uint64_t)(k4 * 2), wide ? IDESC2 : IDESC, (kb | k4) != 0);
        if (x_lo && !wide) {
          const uint64_t xl = umma_desc_k128(base + XLO_OFF);
#pragma unroll
          for (int k4 = 0; k4 < GBK / 16; ++k4) umma_f16(tmem_base, wd + (uint64_t)(k4 * 2), xl + (uint64_t)(k4 * 2), IDESC, 1u);
        }
        if (w_lo) {
          const uint64_t wl = umma_desc_k128(base + G_A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < GBK / 16; ++k4) umma_f16(tmem_base, wl + (uint64_t)(k4 * 2), xd + (uint64_t)(k4 * 2), IDESC, 1u);
        }
        umma_commit(&empty[s]);
      }
      umma_commit(acc_full);
    }
  } else {
    const int quad = warp & 3;
    const int ch = tile_n * GBM + quad * 32 + lane;
    pdl_wait();
    const bool ok = mbar_wait(acc_full, 0, abort_flag, g.status, ST_GEMM_TIMEOUT);
    tc_fence_after();
    if (ok) {
      const float sc = (g.col_scale && ch < g.N && grp.split == 1) ? __half2float(g.col_scale[ch]) : 1.f;
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (m0 + c0 >= g.M) break;   // warp-uniform
        uint32_t acc[32];
        __syncwarp();
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, acc);
        if (FUSE_LO && x_lo) {
          uint32_t part[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(BN + c0), part);
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) + __uint_as_float(part[i]));
        }
        if (ch < g.N) {
          if (grp.split > 1) {
            float *dst = g.raw + ((size_t)blockIdx.z * g.M + m0 + c0) * g.N + ch;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (m0 + c0 + i < g.M) dst[(size_t)i * g.N] = __uint_as_float(acc[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (m0 + c0 + i < g.M) epi_store_one(g, m0 + c0 + i, ch, __uint_as_float(acc[i]) * sc);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// The few-row GEMM for quantised weights: the weight operand is read in its packed form (int8 codes [N, K], or int4
// nibbles [N, K/2] with fp16 group scales [N, K/32]: the bytes a step has to stream) and expanded to the K-major fp16
// tile the tensor core wants inside the kernel, by eight warps that do nothing else.  Per K slice of 64 inputs:
//   warp 0      TMA: packed weights into a ring of slots of their own (128 rows x 32..128 bytes = 1, 2 or 4 slices
//               per slot) and the X tile(s) into buffer kb % NE
//   warps 6..13 expanders (two threads per row): packed slice -> 128 x 64 fp16 in the 128-byte-swizzled layout of a
//               TMA-loaded tile, expanded buffer kb % NE
//               (int8: the integer code, exact in fp16, the row scale is applied to the accumulator;
//                int4: hi = fp16(q * scale) and lo = q * scale - hi, an exact pair)
//   warp 1      MMA: acc += W_hi [X_hi | X_lo] (+ W_lo X_hi)
//   warps 2..5  epilogue, as in gemm_wt_kernel
// Buffer e (its X slot and its expanded weights) is free again when the MMAs that read it have retired: one commit
// per slice.  A weight slot is free when the expanders have read its last slice.  Shared-memory writes of the
// expanders are made visible to the tensor core's (asynchronous) reads with fence.proxy.async before the barrier
// arrive.  The weights are constants, so their loads and their expansion do not wait for the kernels before this
// one: under programmatic dependent launch the first slices are ready when X arrives.
constexpr int WQ_MAX_E = 4;        // most buffers (expanded weights + X)
constexpr int WQ_MAX_W = 8;        // deepest ring of packed weight slots
constexpr int WQ_EXP_WARPS = 8;
constexpr int WQ_THREADS = 192 + 32 * WQ_EXP_WARPS;

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// 72 registers: two CTAs share an SM whenever the launcher's shared-memory plan allows it
template <int BN, int FMT>
__global__ void __launch_bounds__(WQ_THREADS, 2)
gemm_wq_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ GemmGroup grp) {
  constexpr uint32_t X_BYTES = BN * GBK * 2;
  constexpr uint32_t ROW_B = FMT == FMT_INT8 ? GBK : GBK / 2;                  // packed bytes per row and K slice: 64 / 32
  constexpr uint32_t E_BYTES = (FMT == FMT_INT4 ? 2u : 1u) * G_A_BYTES;        // expanded weights: hi (+ lo)
  // Up to 128 rows the hi and lo halves of X sit back to back in a buffer and are one B operand of 2 BN rows: one MMA
  // gives W X_hi in accumulator columns [0, BN) and W X_lo in [BN, 2 BN), which the epilogue adds up.  An MMA with
  // few columns costs about as much as a wide one (it reads the whole 128-row weight operand either way), so this
  // takes a third (int4) or half (int8) of the MMAs off the issue thread.  At 256 rows the halves are passes of their own.
  constexpr bool FUSE_LO = BN <= 128;
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GBM >> 4) << 24);
  constexpr uint32_t IDESC2 = (1u << 4) | ((uint32_t)((2 * BN) >> 3) << 17) | ((uint32_t)(GBM >> 4) << 24);
  constexpr uint32_t TMEM_COLS = FUSE_LO ? 2 * BN : BN;
  // weight slot: 128 rows x WB bytes = KSUB consecutive K slices of the tile; WB = 128 (swizzled like every 128-byte
  // tile: whole lines for the TMA unit and for HBM) where shared memory allows, else 64 or 32 (plain rows)
  const uint32_t WB = grp.wbox, WS_BYTES = GBM * WB;
  const int KSUB = (int)(WB / ROW_B), KSH = KSUB == 4 ? 2 : KSUB == 2 ? 1 : 0;
  const int NW = grp.stages, NE = grp.estages;
  const uint32_t XS_BYTES = grp.stage_bytes;                                   // X part of a buffer: hi (+ lo)
  extern __shared__ uint8_t gsm_raw[];
  uint8_t *gsm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *wfull = reinterpret_cast<uint64_t *>(gsm);
  uint64_t *wempty = wfull + WQ_MAX_W;
  uint64_t *xfull = wempty + WQ_MAX_W;
  uint64_t *a_full = xfull + WQ_MAX_E;
  uint64_t *a_empty = a_full + WQ_MAX_E;
  uint64_t *acc_full = a_empty + WQ_MAX_E;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t etiles = smem_u32(gsm + 1024);                                // NE expanded buffers, 1024-byte aligned
  const uint32_t xtiles = etiles + (uint32_t)NE * E_BYTES;                     // NE X slots
  const uint32_t wtiles = xtiles + (uint32_t)NE * XS_BYTES;                    // NW weight slots
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pi = 0;
  while (pi + 1 < grp.n && (int)blockIdx.x >= grp.tile_start[pi + 1]) ++pi;
  const GemmArgs &g = grp.p[pi];
  const int tile_n = blockIdx.x - grp.tile_start[pi], m0 = blockIdx.y * BN;
  const int num_k1 = g.K / GBK;
  const int kz0 = (int)((long long)blockIdx.z * num_k1 / grp.split), nkz = (int)((long long)(blockIdx.z + 1) * num_k1 / grp.split) - kz0;
  const bool x_lo = g.A2 != nullptr;
  // this CTA's slices [kz0, kz0 + nkz) touch weight slots g0 .. g0 + ng - 1 of the matrix
  const int g0 = kz0 >> KSH, ng = nkz > 0 ? ((kz0 + nkz - 1) >> KSH) - g0 + 1 : 0;

  if (threadIdx.x == 64) { prefetch_tmap(&maps.b[pi]); prefetch_tmap(&maps.a[pi]); if (x_lo) prefetch_tmap(&maps.a2[pi]); }
  if (threadIdx.x == 0) {
    for (int s = 0; s < NW; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wempty[s], WQ_EXP_WARPS); }
    for (int e = 0; e < NE; ++e) { mbar_init(&xfull[e], 1); mbar_init(&a_full[e], WQ_EXP_WARPS); mbar_init(&a_empty[e], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();
  // What the kernels before this one wrote (X, the epilogue's inputs and outputs) is touched only after pdl_wait():
  // by the X loads and by the epilogue warps.

  if (warp == 0) {
    if (lane == 0) {
      // one thread feeds both rings: whichever has a free slot gets its next tile
      int kw = 0, kx = 0, idle = 0;
      unsigned long long t0 = 0;
      for (; kw < ng && kw < NW; ++kw) {
        mbar_expect_tx(&wfull[kw], WS_BYTES);
        tma_load_2d(wtiles + (uint32_t)kw * WS_BYTES, &maps.b[pi], (g0 + kw) * (int)WB, tile_n * GBM, &wfull[kw]);
      }
      pdl_wait();
      while (kw < ng || kx < nkz) {
        bool moved = false;
        if (kw < ng && mbar_try(&wempty[kw % NW], ((kw / NW) & 1) ^ 1)) {
          const int s = kw % NW;
          mbar_expect_tx(&wfull[s], WS_BYTES);
          tma_load_2d(wtiles + (uint32_t)s * WS_BYTES, &maps.b[pi], (g0 + kw) * (int)WB, tile_n * GBM, &wfull[s]);
          ++kw;
          moved = true;
        }
        if (kx < nkz && mbar_try(&a_empty[kx % NE], ((kx / NE) & 1) ^ 1)) {
          const int e = kx % NE;
          const uint32_t dst = xtiles + (uint32_t)e * XS_BYTES;
          const int kc = (kz0 + kx) * GBK;
          mbar_expect_tx(&xfull[e], (x_lo ? 2u : 1u) * X_BYTES);
          tma_load_2d(dst, &maps.a[pi], kc, m0, &xfull[e]);
          if (x_lo) tma_load_2d(dst + X_BYTES, &maps.a2[pi], kc, m0, &xfull[e]);
          ++kx;
          moved = true;
        }
        if (moved) { idle = 0; continue; }
        if (idle == 0) t0 = globaltimer_ns();
        if ((++idle & 63) == 0) {
          if (*abort_flag) break;
          if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; atomicCAS(g.status, 0, ST_GEMM_TIMEOUT); break; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < nkz; ++kb) {
        const int e = kb % NE;
        const uint32_t par = (uint32_t)(kb / NE) & 1u;
        if (!mbar_wait(&xfull[e], par, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
        if (!mbar_wait(&a_full[e], par, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
        tc_fence_after();
        const uint32_t xb = xtiles + (uint32_t)e * XS_BYTES, eb = etiles + (uint32_t)e * E_BYTES;
        const uint64_t wd = umma_desc_k128(eb), xd = umma_desc_k128(xb);
        const bool wide = FUSE_LO && x_lo;
#pragma unroll
        for (int k4 = 0; k4 < GBK / 16; ++k4)
          umma_f16(tmem_base, wd + (uint64_t)(k4 * 2), xd + (uint64_t)(k4 * 2), wide ? IDESC2 : IDESC, (kb | k4) != 0);
        if (x_lo && !wide) {
          const uint64_t xl = umma_desc_k128(xb + X_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < GBK / 16; ++k4) umma_f16(tmem_base, wd + (uint64_t)(k4 * 2), xl + (uint64_t)(k4 * 2), IDESC, 1u);
        }
        if (FMT == FMT_INT4) {
          const uint64_t wl = umma_desc_k128(eb + G_A_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < GBK / 16; ++k4) umma_f16(tmem_base, wl + (uint64_t)(k4 * 2), xd + (uint64_t)(k4 * 2), IDESC, 1u);
        }
        umma_commit(&a_empty[e]);   // X slot e and expanded buffer e are free once these MMAs have retired
      }
      umma_commit(acc_full);
    }
  } else if (warp >= 6) {
    // expanders: two threads per row of the tile, each expands half of the row's 64 inputs
    const int et = (int)threadIdx.x - 192;
    const int row = et >> 1, part = et & 1;
    const int ch = tile_n * GBM + row;                      // output channel of this row
    const uint32_t swz = (uint32_t)(row & 7);
    const uint32_t wswz = WB == 128u ? swz : 0u;
    const uint32_t erow = (uint32_t)row * 128u;             // byte offset of the row inside an expanded tile
    // int4: this row's group scales, two per K slice.  They come straight from global memory, 16 bytes (four slices)
    // at a time and four slices ahead of their use, so that the expansion never waits for them; rows whose scales
    // are not 16-byte aligned (K not a multiple of 256) take them slice by slice, one ahead.
    const __half *gs = nullptr;
    if (FMT == FMT_INT4 && ch < g.N) gs = g.wq_scale + (size_t)ch * (g.K / 32);
    const bool quads = FMT == FMT_INT4 && ((g.K / 32) & 7) == 0;
    const int nquads = g.K / 256;
    uint4 scq = make_uint4(0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u), scq_next = scq;
    uint32_t sc_next = 0x3c003c00u;
    if (FMT == FMT_INT4 && gs && nkz > 0) {
      if (quads) {
        scq = *reinterpret_cast<const uint4 *>(gs + (size_t)(kz0 >> 2) * 8);
        if ((kz0 >> 2) + 1 < nquads) scq_next = *reinterpret_cast<const uint4 *>(gs + (size_t)((kz0 >> 2) + 1) * 8);
      } else {
        sc_next = *reinterpret_cast<const uint32_t *>(gs + (size_t)kz0 * 2);
      }
    }
    for (int kb = 0; kb < nkz; ++kb) {
      const int ks = kz0 + kb;
      const int wj = (ks >> KSH) - g0, sub = ks & (KSUB - 1);
      const int s = wj % NW, e = kb % NE;
      uint32_t sc = sc_next;                                // scales of the two 32-input groups of this slice
      if (FMT == FMT_INT4) {
        if (quads) {
          if (kb > 0 && (ks & 3) == 0) {
            scq = scq_next;
            if (gs && (ks >> 2) + 1 < nquads) scq_next = *reinterpret_cast<const uint4 *>(gs + (size_t)((ks >> 2) + 1) * 8);
          }
          const int qi = ks & 3;
          sc = qi == 0 ? scq.x : qi == 1 ? scq.y : qi == 2 ? scq.z : scq.w;
        } else if (gs && kb + 1 < nkz) {
          sc_next = *reinterpret_cast<const uint32_t *>(gs + (size_t)(ks + 1) * 2);
        }
      }
      if (!mbar_wait(&wfull[s], (uint32_t)(wj / NW) & 1u, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
      if (!mbar_wait(&a_empty[e], ((uint32_t)(kb / NE) & 1u) ^ 1u, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
      // 16-byte chunk c of the row's WB bytes is at (c ^ wswz) << 4
      const uint32_t src = wtiles + (uint32_t)s * WS_BYTES + (uint32_t)row * WB;
      const uint32_t c0 = (uint32_t)sub * (ROW_B / 16u);
      const uint32_t dst = etiles + (uint32_t)e * E_BYTES + erow;
      if (FMT == FMT_INT8) {
        // two 16-byte pieces of 16 codes per thread; neighbouring rows take theirs in opposite order, which spreads a
        // quarter warp's stores over all eight 16-byte columns of the swizzled rows
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
          const uint32_t piece = (uint32_t)part * 2u + ((uint32_t)(pp + row) & 1u);
          const uint4 w = lds128(src + (((c0 + piece) ^ wswz) << 4));
          const uint32_t M = 0x64646464u, OFF = 0x64806480u;    // 1024 + (code + 128) - 1152 = code
          const uint32_t wx = w.x ^ 0x80808080u, wy = w.y ^ 0x80808080u, wz = w.z ^ 0x80808080u, ww = w.w ^ 0x80808080u;
          const uint4 o0 = make_uint4(hsub2_u32(prmt(wx, M, 0x4140), OFF), hsub2_u32(prmt(wx, M, 0x4342), OFF),
                                      hsub2_u32(prmt(wy, M, 0x4140), OFF), hsub2_u32(prmt(wy, M, 0x4342), OFF));
          const uint4 o1 = make_uint4(hsub2_u32(prmt(wz, M, 0x4140), OFF), hsub2_u32(prmt(wz, M, 0x4342), OFF),
                                      hsub2_u32(prmt(ww, M, 0x4140), OFF), hsub2_u32(prmt(ww, M, 0x4342), OFF));
          sts128(dst + (((piece * 2u) ^ swz) << 4), o0);        // inputs 16 piece .. +7: 16-byte chunk 2 piece
          sts128(dst + (((piece * 2u + 1u) ^ swz) << 4), o1);
        }
      } else {
        // one 16-byte piece of 32 nibbles per thread = one of the two scale groups of the slice
        const uint4 w = lds128(src + (((c0 + (uint32_t)part) ^ wswz) << 4));
        const uint32_t s16 = part ? (sc >> 16) : (sc & 0xffffu);
        const uint32_t s2 = s16 | (s16 << 16);
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          // 8 nibbles = 8 consecutive inputs -> one 16-byte chunk of hi and one of lo
          uint32_t hi[4], lo[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // byte j -> {1024 + low nibble, 64 + high nibble} - {1032, 72} = {q_even, q_odd}
            const uint32_t x = prmt(words[wi], 0u, 0x4040u + (uint32_t)j * 0x0101u);   // bytes [b_j, 0, b_j, 0]
            const uint32_t qv = hsub2_u32(lop3_and_or(x, 0x00f0000fu, 0x54006400u), 0x54806408u);
            hi[j] = hmul2_u32(qv, s2);
            lo[j] = hfma2_u32(qv, s2, hi[j] ^ 0x80008000u);
          }
          const uint32_t chunk = ((uint32_t)part * 4u + (uint32_t)wi) ^ swz;
          sts128(dst + (chunk << 4), make_uint4(hi[0], hi[1], hi[2], hi[3]));
          sts128(dst + G_A_BYTES + (chunk << 4), make_uint4(lo[0], lo[1], lo[2], lo[3]));
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&a_full[e]);
        if (sub == KSUB - 1 || kb == nkz - 1) mbar_arrive(&wempty[s]);   // last slice of the slot this CTA uses
      }
    }
  } else {
    const int quad = warp & 3;
    const int ch = tile_n * GBM + quad * 32 + lane;
    pdl_wait();
    const bool ok = mbar_wait(acc_full, 0, abort_flag, g.status, ST_GEMM_TIMEOUT);
    tc_fence_after();
    if (ok) {
      const float sc = (g.col_scale && ch < g.N && grp.split == 1) ? __half2float(g.col_scale[ch]) : 1.f;
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (m0 + c0 >= g.M) break;   // warp-uniform
        uint32_t acc[32];
        __syncwarp();
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, acc);
        if (FUSE_LO && x_lo) {
          uint32_t part[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(BN + c0), part);
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) + __uint_as_float(part[i]));
        }
        if (ch < g.N) {
          if (grp.split > 1) {
            float *dst = g.raw + ((size_t)blockIdx.z * g.M + m0 + c0) * g.N + ch;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (m0 + c0 + i < g.M) dst[(size_t)i * g.N] = __uint_as_float(acc[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (m0 + c0 + i < g.M) epi_store_one(g, m0 + c0 + i, ch, __uint_as_float(acc[i]) * sc);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// split-K: sum the slabs in a fixed order, then the same epilogue.  One thread per 4 consecutive columns of a row
// (coalesced 16-byte reads of every slab); N is a multiple of 4 for every projection (the head never splits).
// blockIdx.y picks the problem of the group (grid.x covers the largest one).
__global__ void __launch_bounds__(256) gemm_finish_kernel(const __grid_constant__ GemmGroup grp) {
  pdl_trigger();
  pdl_wait();
  const GemmArgs &g = grp.p[blockIdx.y];
  const int split = grp.split;
  const int n4 = g.N >> 2;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= g.M * n4) return;
  const int row = idx / n4, col = (idx - row * n4) * 4;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int z = 0; z < split; ++z) {
    const float4 p = *reinterpret_cast<const float4 *>(g.raw + ((size_t)z * g.M + row) * g.N + col);
    v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
  }
  if (g.col_scale) {
    v.x *= __half2float(g.col_scale[col]); v.y *= __half2float(g.col_scale[col + 1]);
    v.z *= __half2float(g.col_scale[col + 2]); v.w *= __half2float(g.col_scale[col + 3]);
  }
  const size_t o = (size_t)row * g.ldo + col;
  float a[4] = {v.x, v.y, v.z, v.w};
  if (g.epi == GEMM_EPI_F32) {
    *reinterpret_cast<float4 *>(reinterpret_cast<float *>(g.out) + o) = v;
  } else if (g.epi == GEMM_EPI_ADD_F32 || g.epi == GEMM_EPI_MULADD_F32) {
    const float4 x = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(g.aux0) + o);
    float r[4] = {1.f, 1.f, 1.f, 1.f};
    if (g.epi == GEMM_EPI_MULADD_F32) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        r[i] = __half2float(reinterpret_cast<const __half *>(g.aux1)[o + i]);
        if (g.aux1_lo) r[i] += __half2float(reinterpret_cast<const __half *>(g.aux1_lo)[o + i]);
      }
    }
    *reinterpret_cast<float4 *>(reinterpret_cast<float *>(g.out) + o) =
        make_float4((x.x + r[0] * a[0]) * g.scale, (x.y + r[1] * a[1]) * g.scale, (x.z + r[2] * a[2]) * g.scale,
                    (x.w + r[3] * a[3]) * g.scale);
  } else {
    __half *out = reinterpret_cast<__half *>(g.out) + o;
    __half *lo = g.out_lo ? reinterpret_cast<__half *>(g.out_lo) + o : nullptr;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float e = epi_half_op(g.epi, a[i]);
      const __half h = __float2half_rn(e);
      out[i] = h;
      if (lo) lo[i] = __float2half_rn(e - __half2float(h));
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, K] fp16 row-major -> tensor map with a (64 x box_rows) box, 128-byte swizzle, zero fill outside
bool make_map(CUtensorMap *map, const void *base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)GBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [rows, row_bytes] bytes row-major -> tensor map with a (box_bytes x 128 rows) box, zero fill outside; 128-byte boxes
// are swizzled, narrower ones are plain rows
bool make_map_bytes(CUtensorMap *map, const void *base, int rows, int row_bytes, int box_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)GBM};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

namespace {
// [K, N] -> [N, K], 32 x 32 tiles through shared memory
__global__ void transpose_f16_kernel(const __half *src, int K, int N, __half *dst) {
  __shared__ __half tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    if (k < K && n < N) tile[r][threadIdx.x] = src[(size_t)k * N + n];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (k < K && n < N) dst[(size_t)n * K + k] = tile[threadIdx.x][r];
  }
}
}  // namespace

cudaError_t launch_transpose_f16(const __half *src, int K, int N, __half *dst, cudaStream_t st) {
  dim3 grid((N + 31) / 32, (K + 31) / 32), block(32, 8);
  transpose_f16_kernel<<<grid, block, 0, st>>>(src, K, N, dst);
  return cudaGetLastError();
}

namespace {

// ---- block reductions (blockDim.x = 256) -------------------------------------------------------------
__device__ __forceinline__ float2 block_sum2(float a, float b, float *red /* [16] */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();   // red may still be read from the previous call
  if (lane == 0) { red[warp * 2] = a; red[warp * 2 + 1] = b; }
  __syncthreads();
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) { sa += red[w * 2]; sb += red[w * 2 + 1]; }
  return make_float2(sa, sb);
}

// mean and 1/std of one fp32 row (shifted single pass, like the decode prologue)
__device__ __forceinline__ float2 row_stats(const float *x, int C, float *red) {
  const float piv = x[0];
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const float d = x[i] - piv;
    s1 += d; s2 += d * d;
  }
  const float2 s = block_sum2(s1, s2, red);
  const float m = s.x / (float)C;
  float var = s.y / (float)C - m * m;
  var = var > 0.f ? var : 0.f;
  return make_float2(piv + m, rsqrtf(var + 1e-5f));
}

// x[t, :] = embedding row of ids[t]
__global__ void gather_emb_kernel(const void *emb, int emb_f32, const int32_t *ids, int C, float *x) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t row = (size_t)ids[t] * C;
  for (int i = threadIdx.x; i < C; i += blockDim.x)
    x[(size_t)t * C + i] = emb_f32 ? reinterpret_cast<const float *>(emb)[row + i]
                                   : __half2float(reinterpret_cast<const __half *>(emb)[row + i]);
}

// LayerNorm + token shift + mix for every token row (LN of att_seq.cu:375, the shifted cat of :377-381 and the
// MixWithG of :384; ffn_seq.cu:70-76): op_v[t] = xx[t] * mu_v + prev[t] * (1 - mu_v), prev[0] = the stored shift
// state, prev[t] = xx[t-1]; the new shift state is xx[T-1].  One CTA per token; it normalises its own row and the
// row before it, so no CTA waits for another.
// Batch mode (rows = independent streams, one token each): prev of row b is stream b's stored shift state and every
// row writes its new one.  nvec == 0: plain LayerNorm into op[0] (ln_out before the head).
// Each thread keeps its float4 pieces of the row (and of the row before) in registers: x is read once.
constexpr int LN_MAX4 = 8;   // float4 per thread: n_embd <= 8192
template <int NJ>
__device__ __forceinline__ float2 stats_from_regs(const float4 *v, int n4, float piv, int C, float *red) {
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    if ((int)threadIdx.x + j * 256 < n4) {
      const float d0 = v[j].x - piv, d1 = v[j].y - piv, d2 = v[j].z - piv, d3 = v[j].w - piv;
      s1 += (d0 + d1) + (d2 + d3);
      s2 += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  const float2 s = block_sum2(s1, s2, red);
  const float m = s.x / (float)C;
  float var = s.y / (float)C - m * m;
  var = var > 0.f ? var : 0.f;
  return make_float2(piv + m, rsqrtf(var + 1e-5f));
}
__device__ __forceinline__ void store_hl4(__half *hi, __half *lo, size_t o, const float4 &v) {
  const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t *>(&h0); u.y = *reinterpret_cast<const uint32_t *>(&h1);
  *reinterpret_cast<uint2 *>(hi + o) = u;
  if (lo) {
    const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
    const __half2 l0 = __floats2half2_rn(v.x - f0.x, v.y - f0.y), l1 = __floats2half2_rn(v.z - f1.x, v.w - f1.y);
    u.x = *reinterpret_cast<const uint32_t *>(&l0); u.y = *reinterpret_cast<const uint32_t *>(&l1);
    *reinterpret_cast<uint2 *>(lo + o) = u;
  }
}
__device__ __forceinline__ float4 load_act_f4(const void *p, int i4, int act_fp16) {
  if (act_fp16) {
    const uint2 u = reinterpret_cast<const uint2 *>(p)[i4];
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  return reinterpret_cast<const float4 *>(p)[i4];
}
__device__ __forceinline__ float round_h(float v) { return __half2float(__float2half_rn(v)); }

// NJ = float4 pieces of a row per thread (2, 4 or 8: n_embd up to 2048, 4096, 8192)
template <int NJ>
__global__ void __launch_bounds__(256) ln_mix_seq_kernel(SeqLnArgs a) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[16];
  const int t = blockIdx.x, C = a.C, n4 = C >> 2;
  const float4 *xr = reinterpret_cast<const float4 *>(a.x + (size_t)t * C);
  const bool from_row = !a.batch_mode && t > 0 && a.nvec > 0;
  float4 xv[NJ], pv[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int i4 = threadIdx.x + j * 256;
    if (i4 < n4) {
      xv[j] = xr[i4];
      if (from_row) pv[j] = xr[i4 - n4];
    }
  }
  float piv = a.x[(size_t)t * C];
  if (a.pend_split > 1) {
    // the projection before this LayerNorm left its split-K slabs: sum them (in slab order, like gemm_finish_kernel),
    // apply its epilogue x = (x + [r *] sum) * scale, store the finished row and normalise it from the registers
    __shared__ float piv_s;
    float4 acc[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    const size_t zs = (size_t)a.T * C;
    constexpr int ZB = NJ <= 2 ? 8 : 4;   // slabs per batch: NJ x ZB 16-byte loads in flight per thread
    for (int z0 = 0; z0 < a.pend_split; z0 += ZB) {
      float4 p[NJ][ZB];
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int i4 = threadIdx.x + j * 256;
        const float *slab = a.pend_raw + (size_t)t * C + (size_t)i4 * 4;
#pragma unroll
        for (int i = 0; i < ZB; ++i)
          if (i4 < n4 && z0 + i < a.pend_split) p[j][i] = *reinterpret_cast<const float4 *>(slab + (size_t)(z0 + i) * zs);
      }
#pragma unroll
      for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int i = 0; i < ZB; ++i)   // in slab order
          if (z0 + i < a.pend_split) { acc[j].x += p[j][i].x; acc[j].y += p[j][i].y; acc[j].z += p[j][i].z; acc[j].w += p[j][i].w; }
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      const int i4 = threadIdx.x + j * 256;
      if (i4 >= n4) continue;
      float4 v = acc[j];
      if (a.pend_cscale) {
        const __half *cs = a.pend_cscale + (size_t)i4 * 4;
        v.x *= __half2float(cs[0]); v.y *= __half2float(cs[1]); v.z *= __half2float(cs[2]); v.w *= __half2float(cs[3]);
      }
      float r[4] = {1.f, 1.f, 1.f, 1.f};
      if (a.pend_r) {
        const size_t o = (size_t)t * C + (size_t)i4 * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          r[i] = __half2float(a.pend_r[o + i]);
          if (a.pend_r_lo) r[i] += __half2float(a.pend_r_lo[o + i]);
        }
      }
      xv[j] = make_float4((xv[j].x + r[0] * v.x) * a.pend_scale, (xv[j].y + r[1] * v.y) * a.pend_scale,
                          (xv[j].z + r[2] * v.z) * a.pend_scale, (xv[j].w + r[3] * v.w) * a.pend_scale);
      reinterpret_cast<float4 *>(a.x_wr + (size_t)t * C)[i4] = xv[j];
      if (i4 == 0) piv_s = xv[j].x;
    }
    __syncthreads();
    piv = piv_s;
  }
  const float2 st = stats_from_regs<NJ>(xv, n4, piv, C, red);
  float2 sp = make_float2(0.f, 0.f);
  if (from_row) sp = stats_from_regs<NJ>(pv, n4, a.x[(size_t)(t - 1) * C], C, red);
  const uint8_t *srd = reinterpret_cast<const uint8_t *>(a.sx_rd) + (a.batch_mode ? (size_t)t * a.state_stride : 0);
  uint8_t *swr = reinterpret_cast<uint8_t *>(a.sx_wr) + (a.batch_mode ? (size_t)t * a.state_stride : 0);
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int i4 = threadIdx.x + j * 256;
    if (i4 >= n4) continue;
    const float4 w = reinterpret_cast<const float4 *>(a.ln_w)[i4], b = reinterpret_cast<const float4 *>(a.ln_b)[i4];
    const float4 xx = make_float4((xv[j].x - st.x) * st.y * w.x + b.x, (xv[j].y - st.x) * st.y * w.y + b.y,
                                  (xv[j].z - st.x) * st.y * w.z + b.z, (xv[j].w - st.x) * st.y * w.w + b.w);
    const size_t o = (size_t)t * C + (size_t)i4 * 4;
    if (a.nvec == 0) {
      store_hl4(a.op[0], a.op_lo[0], o, xx);
      continue;
    }
    float4 prev;
    if (from_row) {
      prev = make_float4((pv[j].x - sp.x) * sp.y * w.x + b.x, (pv[j].y - sp.x) * sp.y * w.y + b.y,
                         (pv[j].z - sp.x) * sp.y * w.z + b.z, (pv[j].w - sp.x) * sp.y * w.w + b.w);
      // what the token loop would have stored as shift state
      if (a.act_fp16) prev = make_float4(round_h(prev.x), round_h(prev.y), round_h(prev.z), round_h(prev.w));
    } else {
      prev = load_act_f4(srd, i4, a.act_fp16);
    }
#pragma unroll
    for (int v = 0; v < 4; ++v)
      if (v < a.nvec) {
        const float4 m = reinterpret_cast<const float4 *>(a.mix[v])[i4];
        store_hl4(a.op[v], a.op_lo[v], o,
                  make_float4(xx.x * m.x + prev.x * (1.f - m.x), xx.y * m.y + prev.y * (1.f - m.y),
                              xx.z * m.z + prev.z * (1.f - m.z), xx.w * m.w + prev.w * (1.f - m.w)));
      }
    if (a.batch_mode || t == a.T - 1) {
      if (a.act_fp16) {
        const __half2 h0 = __floats2half2_rn(xx.x, xx.y), h1 = __floats2half2_rn(xx.z, xx.w);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t *>(&h0); u.y = *reinterpret_cast<const uint32_t *>(&h1);
        reinterpret_cast<uint2 *>(swr)[i4] = u;
      } else {
        reinterpret_cast<float4 *>(swr)[i4] = xx;
      }
    }
  }
}

// RWKV-4 WKV over rows (WkvForwardOne, att.cu:30-62, with the sigmoid of att.cu:154-159 fused): one thread per
// (stream, channel).  Seq mode: one stream, T rows in order; batch mode: row b is the one token of stream b.
//   out[row, c] = sigmoid(r) * wkv (fp16, the operand of the output projection); aa, bb, pp updated in place.
__global__ void __launch_bounds__(256) wkv4_rows_kernel(Wkv4Args a) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= a.C) return;
  float *st = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(a.state) + (size_t)b * a.state_stride);
  float aa = st[c], bb = st[a.C + c], pp = st[2 * a.C + c];
  const float u = a.first[c], w = a.decay[c];
  const int t0 = a.batch_mode ? b : 0, t1 = a.batch_mode ? b + 1 : a.T;
  for (int t = t0; t < t1; ++t) {
    const size_t o = (size_t)t * a.C + c;
    float k, v, rp;
    if (a.split > 1) {
      // the projections left their split-K slabs: sum them here, in slab order like gemm_finish_kernel
      k = 0.f; v = 0.f; rp = 0.f;
      for (int z = 0; z < a.split; ++z) {
        const size_t zo = ((size_t)z * a.T + t) * a.C + c;
        k += a.raw_k[zo]; v += a.raw_v[zo]; rp += a.raw_r[zo];
      }
      if (a.cs_k) { k *= __half2float(a.cs_k[c]); v *= __half2float(a.cs_v[c]); rp *= __half2float(a.cs_r[c]); }
    } else {
      k = a.k[o]; v = a.v[o]; rp = a.r[o];
    }
    const float r = 1.f / (1.f + expf(-rp));
    float ww = u + k;
    float pm = fmaxf(pp, ww);
    float e1 = expf(pp - pm), e2 = expf(ww - pm);
    const float wkv = (e1 * aa + e2 * v) / (e1 * bb + e2);
    const __half oh = __float2half_rn(r * wkv);
    a.out[o] = oh;
    if (a.out_lo) a.out_lo[o] = __float2half_rn(r * wkv - __half2float(oh));
    ww = w + pp;
    pm = fmaxf(ww, k);
    e1 = expf(ww - pm);
    e2 = expf(k - pm);
    aa = e1 * aa + e2 * v;
    bb = e1 * bb + e2;
    pp = pm;
  }
  st[c] = aa; st[a.C + c] = bb; st[2 * a.C + c] = pp;
}

// greedy sample of every row: index of the largest logit (lowest index on ties).  ctl (optional): the id also goes
// to row ctl->step of the history ctl->hist -- fixed kernel arguments, so that a captured graph can be replayed.
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float *logits, int V, int ld, int32_t *out, const GreedyCtl *ctl) {
  pdl_trigger();
  pdl_wait();
  __shared__ unsigned long long best[8];
  const float *row = logits + (size_t)blockIdx.x * ld;
  unsigned long long m = 0;
  auto take = [&](float f, int i) {
    unsigned u = __float_as_uint(f);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    const unsigned long long w = ((unsigned long long)u << 32) | (0xffffffffu - (unsigned)i);
    m = w > m ? w : m;
  };
  const int V4 = ((ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) ? (V & ~3) : 0;
  // 16-byte loads, eight in flight per thread: a row is read by one CTA, so the loads in flight set its speed
#pragma unroll 8
  for (int i = threadIdx.x * 4; i < V4; i += blockDim.x * 4) {
    const float4 f = *reinterpret_cast<const float4 *>(row + i);
    take(f.x, i); take(f.y, i + 1); take(f.z, i + 2); take(f.w, i + 3);
  }
  for (int i = V4 + threadIdx.x; i < V; i += blockDim.x) take(row[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, m, o);
    m = other > m ? other : m;
  }
  if ((threadIdx.x & 31) == 0) best[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w8 = 1; w8 < 8; ++w8) m = best[w8] > m ? best[w8] : m;
    const int32_t id = (int32_t)(0xffffffffu - (unsigned)m);
    out[blockIdx.x] = id;
    if (ctl) ctl->hist[(size_t)ctl->step * gridDim.x + blockIdx.x] = id;
  }
}
__global__ void greedy_bump_kernel(GreedyCtl *ctl) { pdl_trigger(); pdl_wait(); ctl->step += 1; }


// RWKV-5 state scan over the tokens of one head (rwkv5_2_kernel_forward, att_seq.cu:258-322; per-head decay for 5.0):
//   y[t, j] = sum_i r[t,i] * (u_i * k[t,i] * v[t,j] + s[i,j]);   s[i,j] = w_i * s[i,j] + k[t,i] * v[t,j]
// r, k, v of 16 tokens at a time arrive in shared memory by cp.async, the next 16 while the current ones are used.
// The sequence is cut into n_chunks pieces that run in parallel (the reference walks it serially):
//   mode 0  state only, from zero, over chunk c               -> E[h][c]        (grid H x n_chunks)
//   mode 1  S_in[h][0] = state; S_in[h][c+1] = w^len(c) * S_in[h][c] + E[h][c]; state = the last one   (grid H)
//   mode 2  full recurrence over chunk c from S_in[h][c]       -> y              (grid H x n_chunks)
// With n_chunks == 1 mode 2 alone reads and writes the model state directly.
constexpr int WKV_TT = 16;

__device__ __forceinline__ void wkv_stage(float (*sr)[64], float (*sk)[64], float (*sv)[64], const SeqWkvArgs &a, int h, int t0,
                                          int nt, bool with_r) {
  // 16 floats = 4 x 16 bytes per (token, vector) quarter row: 3 vectors x nt tokens x 16 pieces
  for (int e = threadIdx.x; e < nt * 16; e += blockDim.x) {
    const int tt = e >> 4, c = (e & 15) * 4;
    const size_t g = (size_t)(t0 + tt) * a.C + h * 64 + c;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&sk[tt][c])), "l"(a.k + g) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&sv[tt][c])), "l"(a.v + g) : "memory");
    if (with_r) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&sr[tt][c])), "l"(a.r + g) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// 64 threads per CTA: thread (jg, iq) owns value columns jg, jg + 16, jg + 32, jg + 48 and key rows 16 iq .. 16 iq + 15,
// i.e. 64 state entries in registers; the r / k values it reads from shared memory serve four columns each.
constexpr int WKV_THREADS = 64;
// Packed fp32 pairs (fma.rn.f32x2 / mul.rn.f32x2: two fp32 operations per instruction on sm_100).  The scan is bound
// by the issue rate of its multiply-adds, so the state is kept as pairs over neighbouring key rows: k, r and the decay
// then come out of shared memory already paired, and only v needs a broadcast pair per token.
__device__ __forceinline__ unsigned long long pack_f2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f2(unsigned long long v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long mul_f2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// y_t[j] = sum_i r_i (u_i k_i v_j + s_ij) = v_j (sum_i r_i u_i k_i) + sum_i r_i s_ij;  s_ij <- w_i s_ij + k_i v_j.
// Thread (jg, iq) owns key rows iq*16 .. +15 of value columns jg + 16 q (q = 0..3): 32 pairs.
template <int MODE>
__global__ void __launch_bounds__(WKV_THREADS) wkv5_seq_kernel(SeqWkvArgs a) {
  pdl_trigger();
  pdl_wait();
  __shared__ __align__(16) float sr[2][WKV_TT][64], sk[2][WKV_TT][64], sv[2][WKV_TT][64];
  const int h = blockIdx.x, c = blockIdx.y, C = a.C;
  const int jg = threadIdx.x >> 2, iq = threadIdx.x & 3;
  // batch mode: blockIdx.y is the stream, its one token is row c, its state lies state_stride floats further
  const int t_begin = a.batch_mode ? c : c * a.chunk_len, t_end = a.batch_mode ? c + 1 : min(a.T, t_begin + a.chunk_len);
  unsigned long long s2[4][8], w2[8], u2[8];   // pairs over key rows (iq*16 + 2 p, + 2 p + 1)
  float *Sown = a.state + (a.batch_mode ? (size_t)c * a.state_stride : 0) + (size_t)h * 4096;
  const float *Sin = a.n_chunks == 1 ? Sown : a.s_in + ((size_t)h * a.n_chunks + c) * 4096;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const int ii = iq * 16 + 2 * p;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      s2[q][p] = MODE == 0 ? 0ull : pack_f2(Sin[ii * 64 + jg + 16 * q], Sin[(ii + 1) * 64 + jg + 16 * q]);
    w2[p] = a.per_head ? pack_f2(a.decay[h], a.decay[h]) : pack_f2(a.decay[h * 64 + ii], a.decay[h * 64 + ii + 1]);
    u2[p] = a.per_head ? pack_f2(a.first[h], a.first[h]) : pack_f2(a.first[h * 64 + ii], a.first[h * 64 + ii + 1]);
  }
  int buf = 0;
  if (t_begin < t_end) wkv_stage(sr[0], sk[0], sv[0], a, h, t_begin, min(WKV_TT, t_end - t_begin), MODE == 2);
  for (int t0 = t_begin; t0 < t_end; t0 += WKV_TT) {
    const int nt = min(WKV_TT, t_end - t0);
    const int tn = t0 + WKV_TT;
    if (tn < t_end) {
      wkv_stage(sr[buf ^ 1], sk[buf ^ 1], sv[buf ^ 1], a, h, tn, min(WKV_TT, t_end - tn), MODE == 2);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      float vj[4];
      unsigned long long v2[4], y2[4] = {0ull, 0ull, 0ull, 0ull}, ruk2 = 0ull;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        vj[q] = sv[buf][tt][jg + 16 * q];
        v2[q] = pack_f2(vj[q], vj[q]);
      }
#pragma unroll
      for (int p = 0; p < 8; p += 2) {
        // four key rows = two pairs per 16-byte load
        const ulonglong2 k4 = *reinterpret_cast<const ulonglong2 *>(&sk[buf][tt][iq * 16 + 2 * p]);
        ulonglong2 r4 = make_ulonglong2(0ull, 0ull);
        if (MODE == 2) r4 = *reinterpret_cast<const ulonglong2 *>(&sr[buf][tt][iq * 16 + 2 * p]);
        const unsigned long long kk[2] = {k4.x, k4.y}, rr[2] = {r4.x, r4.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          if (MODE == 2) ruk2 = fma_f2(mul_f2(rr[e], u2[p + e]), kk[e], ruk2);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (MODE == 2) y2[q] = fma_f2(rr[e], s2[q][p + e], y2[q]);
            s2[q][p + e] = fma_f2(s2[q][p + e], w2[p + e], mul_f2(kk[e], v2[q]));
          }
        }
      }
      if (MODE == 2) {
        float ra, rb;
        unpack_f2(ruk2, ra, rb);
        const float ruk = ra + rb;
        float y[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float ya, yb;
          unpack_f2(y2[q], ya, yb);
          y[q] = fmaf(vj[q], ruk, ya + yb);
          y[q] += __shfl_xor_sync(0xffffffffu, y[q], 1);
          y[q] += __shfl_xor_sync(0xffffffffu, y[q], 2);
        }
        if (iq == 0) {
#pragma unroll
          for (int q = 0; q < 4; ++q) a.y[(size_t)(t0 + tt) * C + h * 64 + jg + 16 * q] = y[q];
        }
      }
    }
    __syncthreads();   // the buffer just read is the one the next staging overwrites
    buf ^= 1;
  }
  if (MODE == 0 || a.n_chunks == 1) {
    float *S = MODE == 0 ? a.e_out + ((size_t)h * a.n_chunks + c) * 4096 : Sown;
#pragma unroll
    for (int p = 0; p < 8; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float lo, hi;
        unpack_f2(s2[q][p], lo, hi);
        const int ii = iq * 16 + 2 * p;
        S[ii * 64 + jg + 16 * q] = lo;
        S[(ii + 1) * 64 + jg + 16 * q] = hi;
      }
  }
}

// mode 1: chain the chunk states; one thread per state entry (grid = H * 16 CTAs of 256 threads), the chunk end
// states are fetched eight at a time ahead of the dependent multiply-adds
__global__ void __launch_bounds__(256) wkv5_combine_kernel(SeqWkvArgs a) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x >> 4, e = (blockIdx.x & 15) * 256 + threadIdx.x;
  const int i = e >> 6;
  const float w = a.per_head ? a.decay[h] : a.decay[h * 64 + i];
  const float lw = log2f(w);
  const float wl = exp2f(lw * (float)a.chunk_len);
  float *S = a.state + (size_t)h * 4096;
  float s = S[e];
  const size_t base = (size_t)h * a.n_chunks * 4096 + e;
  for (int c0 = 0; c0 < a.n_chunks; c0 += 8) {
    float ev[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) ev[q] = c0 + q < a.n_chunks ? a.e_out[base + (size_t)(c0 + q) * 4096] : 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int c = c0 + q;
      if (c < a.n_chunks) {
        a.s_in[base + (size_t)c * 4096] = s;
        const int len = min(a.T, (c + 1) * a.chunk_len) - c * a.chunk_len;
        s = (len == a.chunk_len ? wl : exp2f(lw * (float)len)) * s + ev[q];
      }
    }
  }
  S[e] = s;
}

// GroupNorm over each head's 64 readout values (eps 1e-5, fp32 affine), times the gate where the version has one
// (att_seq.cu:406-415): one warp per (token, head)
__global__ void __launch_bounds__(256) gn_gate_seq_kernel(const float *y, const float *lnx_w, const float *lnx_b, const __half *g,
                                                          const __half *g_lo, int T, int H, __half *out, __half *out_lo) {
  pdl_trigger();
  pdl_wait();
  const int unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (unit >= T * H) return;
  const int t = unit / H, h = unit - t * H;
  const size_t o = (size_t)t * H * 64 + h * 64 + lane * 2;
  const float2 v = *reinterpret_cast<const float2 *>(y + o);
  float s = v.x + v.y;
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
  const float mean = s * (1.f / 64.f);
  const float d0 = v.x - mean, d1 = v.y - mean;
  float q = d0 * d0 + d1 * d1;
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) q += __shfl_xor_sync(0xffffffffu, q, k);
  const float rstd = rsqrtf(q * (1.f / 64.f) + 1e-5f);
  const int c = h * 64 + lane * 2;
  float a0 = d0 * rstd * lnx_w[c] + lnx_b[c], a1 = d1 * rstd * lnx_w[c + 1] + lnx_b[c + 1];
  if (g) {
    float2 gg = __half22float2(*reinterpret_cast<const __half2 *>(g + o));
    if (g_lo) {
      const float2 gl = __half22float2(*reinterpret_cast<const __half2 *>(g_lo + o));
      gg.x += gl.x; gg.y += gl.y;
    }
    a0 *= gg.x; a1 *= gg.y;
  }
  const __half2 hh = __floats2half2_rn(a0, a1);
  *reinterpret_cast<__half2 *>(out + o) = hh;
  if (out_lo) {
    const float2 hf = __half22float2(hh);
    *reinterpret_cast<__half2 *>(out_lo + o) = __floats2half2_rn(a0 - hf.x, a1 - hf.y);
  }
}

// plain LayerNorm of one row -> fp32 vector (ln_out before the head, model_forward_seq.cpp:171-175)
__global__ void __launch_bounds__(256) ln_row_kernel(const float *x, const float *w, const float *b, int C, float *out) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[16];
  const float2 st = row_stats(x, C, red);
  for (int i = threadIdx.x; i < C; i += blockDim.x) out[i] = (x[i] - st.x) * st.y * w[i] + b[i];
}

}  // namespace

cudaError_t launch_gather_emb(const void *emb, int emb_f32, const int32_t *ids, int T, int C, float *x, cudaStream_t st) {
  launch_k(gather_emb_kernel, dim3(T), dim3(256), 0, st, emb, emb_f32, ids, C, x);
  return cudaGetLastError();
}
cudaError_t launch_ln_mix_seq(const SeqLnArgs &a, cudaStream_t st) {
  const int n4 = a.C >> 2;
  if (n4 <= 2 * 256) launch_k(ln_mix_seq_kernel<2>, dim3(a.T), dim3(256), 0, st, a);
  else if (n4 <= 4 * 256) launch_k(ln_mix_seq_kernel<4>, dim3(a.T), dim3(256), 0, st, a);
  else launch_k(ln_mix_seq_kernel<LN_MAX4>, dim3(a.T), dim3(256), 0, st, a);
  return cudaGetLastError();
}
// CTAs of the readout pass of the scan that are resident at once on the device: one wave of (head, chunk) pairs is what
// a prompt should be cut into (a second, partly filled wave costs as much as a full one)
int wkv5_scan_slots() {
  static int slots = 0;
  if (!slots) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, wkv5_seq_kernel<2>, WKV_THREADS, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
    slots = per_sm * device_sm_count();
  }
  return slots;
}

cudaError_t launch_wkv5_seq(const SeqWkvArgs &a, int H, cudaStream_t st) {
  if (a.batch_mode) {
    launch_k(wkv5_seq_kernel<2>, dim3(dim3(H, a.T)), dim3(WKV_THREADS), 0, st, a);   // n_chunks == 1: every stream reads and writes its own state
    return cudaGetLastError();
  }
  if (a.n_chunks <= 1) {
    launch_k(wkv5_seq_kernel<2>, dim3(dim3(H, 1)), dim3(WKV_THREADS), 0, st, a);
    return cudaGetLastError();
  }
  launch_k(wkv5_seq_kernel<0>, dim3(dim3(H, a.n_chunks)), dim3(WKV_THREADS), 0, st, a);
  launch_k(wkv5_combine_kernel, dim3(H * 16), dim3(256), 0, st, a);
  launch_k(wkv5_seq_kernel<2>, dim3(dim3(H, a.n_chunks)), dim3(WKV_THREADS), 0, st, a);
  return cudaGetLastError();
}
cudaError_t launch_wkv4_rows(const Wkv4Args &a, cudaStream_t st) {
  dim3 grid((a.C + 255) / 256, a.batch_mode ? a.T : 1);
  launch_k(wkv4_rows_kernel, dim3(grid), dim3(256), 0, st, a);
  return cudaGetLastError();
}
cudaError_t launch_argmax_rows(const float *logits, int rows, int V, int ld, int32_t *out, GreedyCtl *ctl, cudaStream_t st) {
  launch_k(argmax_rows_kernel, dim3(rows), dim3(256), 0, st, logits, V, ld, out, ctl);
  if (ctl) launch_k(greedy_bump_kernel, dim3(1), dim3(1), 0, st, ctl);
  return cudaGetLastError();
}
cudaError_t launch_gn_gate_seq(const float *y, const float *lnx_w, const float *lnx_b, const __half *g, const __half *g_lo, int T,
                               int H, __half *out, __half *out_lo, cudaStream_t st) {
  launch_k(gn_gate_seq_kernel, dim3((T * H + 7) / 8), dim3(256), 0, st, y, lnx_w, lnx_b, g, g_lo, T, H, out, out_lo);
  return cudaGetLastError();
}
cudaError_t launch_ln_row(const float *x, const float *w, const float *b, int C, float *out, cudaStream_t st) {
  launch_k(ln_row_kernel, dim3(1), dim3(256), 0, st, x, w, b, C, out);
  return cudaGetLastError();
}

namespace {
template <int MT, int BN>
cudaError_t launch_gemm_t(const GemmMaps &maps, const GemmGroup &grp, dim3 grid, size_t smem, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(gemm_f16_kernel<MT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  launch_k(gemm_f16_kernel<MT, BN>, dim3(grid), dim3(G_THREADS), smem, st, maps, grp);
  return cudaGetLastError();
}
}  // namespace

namespace {
template <int BN>
cudaError_t launch_gemm_wt_t(const GemmMaps &maps, const GemmGroup &grp, dim3 grid, size_t smem, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(gemm_wt_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  launch_k(gemm_wt_kernel<BN>, dim3(grid), dim3(G_THREADS), smem, st, maps, grp);
  return cudaGetLastError();
}

// FR_B200_GEMM_WT=0 sends few-row GEMMs through the 64-column tiles of gemm_f16_kernel instead (for comparison)
bool wt_enabled() {
  static const int on = [] { const char *v = getenv("FR_B200_GEMM_WT"); return !(v && v[0] == '0'); }();
  return on != 0;
}

// up to GEMM_SMALL_M rows: weights along the MMA rows (gemm_wt_kernel), split-K into slabs when scratch was given
cudaError_t launch_gemm_wt(const GemmArgs *probs, int n, cudaStream_t st, int *defer_split) {
  const int M = probs[0].M;
  // (measured at 200 .. 512 rows: 256-row X tiles beat two passes with 128-row tiles by 10 %)
  const int bn = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  GemmMaps maps;
  GemmGroup grp;
  memset(&grp, 0, sizeof(grp));
  grp.n = n;
  int tiles = 0, min_k1 = 1 << 30;
  bool raw_ok = true;
  for (int i = 0; i < n; ++i) {
    const GemmArgs &g = probs[i];
    if (g.K % GBK != 0 || g.M < 1 || g.N < 1 || g.M != M) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.Bt) & 15) || (reinterpret_cast<uintptr_t>(g.A2) & 15) ||
        (reinterpret_cast<uintptr_t>(g.Bt2) & 15))
      return cudaErrorInvalidValue;
    if (!make_map(&maps.a[i], g.A, g.M, g.K, bn) || !make_map(&maps.b[i], g.Bt, g.N, g.K, GBM)) return cudaErrorNotSupported;
    if (!make_map(&maps.a2[i], g.A2 ? g.A2 : g.A, g.M, g.K, bn)) return cudaErrorNotSupported;
    if (!make_map(&maps.b2[i], g.Bt2 ? g.Bt2 : g.Bt, g.N, g.K, GBM)) return cudaErrorNotSupported;
    grp.p[i] = g;
    grp.tile_start[i] = tiles;
    tiles += (g.N + GBM - 1) / GBM;
    min_k1 = std::min(min_k1, g.K / GBK);
    raw_ok = raw_ok && g.raw != nullptr && (g.N & 3) == 0 && (g.ldo & 3) == 0;
    if (g.A2) grp.dual |= 1;
    if (g.Bt2) grp.dual |= 2;
  }
  for (int i = n; i < GEMM_GROUP_MAX; ++i) { maps.a[i] = maps.a[0]; maps.a2[i] = maps.a2[0]; maps.b[i] = maps.b[0]; maps.b2[i] = maps.b2[0]; }
  grp.tile_start[n] = tiles;
  const int m_tiles = (M + bn - 1) / bn;
  // one CTA per SM, none waiting for a second wave: split K until the tiles about cover the SMs
  // (up to 64 rows the slabs are small next to the weights and two CTAs fit an SM: twice the slots, so that every SM
  // streams even when the group has few tiles)
  grp.split = 1;
  const int sms = device_sm_count();
  const int slots = bn <= 64 ? 2 * sms : sms;
  if (raw_ok) {
    // cost of a split, in K slices of one CTA: waves x (slices per CTA + fill and drain) + the slabs it adds
    const int ctas = tiles * m_tiles, max_split = std::max(1, std::min(GEMM_SPLIT_MAX, min_k1 / 2));
    float best = 0.f;
    for (int sp = 1; sp <= max_split; ++sp) {
      const int waves = (ctas * sp + slots - 1) / slots;
      const float cost = (float)waves * (float)((min_k1 + sp - 1) / sp + 2) + 0.25f * (float)sp;
      if (sp == 1 || cost < best) { best = cost; grp.split = sp; }
    }
  }
  grp.stage_bytes = ((grp.dual & 2) ? 2u : 1u) * G_A_BYTES + ((grp.dual & 1) ? 2u : 1u) * (uint32_t)bn * GBK * 2;
  // two CTAs per SM with rings of >= 3 slots where they fit (shorter tail when there are more tiles than SMs),
  // else one CTA with as deep a ring as fits
  int stages = (int)((100u << 10) / grp.stage_bytes);
  if (stages < 3) stages = (int)((200u << 10) / grp.stage_bytes);
  grp.stages = std::max(2, std::min(stages, WT_MAX_STAGES));
  const size_t smem = 1024 + (size_t)grp.stages * grp.stage_bytes + 1024;
  dim3 grid(tiles, m_tiles, grp.split);
  cudaError_t e = bn == 32    ? launch_gemm_wt_t<32>(maps, grp, grid, smem, st)
                  : bn == 64  ? launch_gemm_wt_t<64>(maps, grp, grid, smem, st)
                  : bn == 128 ? launch_gemm_wt_t<128>(maps, grp, grid, smem, st)
                              : launch_gemm_wt_t<256>(maps, grp, grid, smem, st);
  if (e != cudaSuccess) return e;
  if (defer_split) *defer_split = grp.split;
  if (grp.split > 1 && !defer_split) {
    int max_n = 0;
    for (int i = 0; i < n; ++i) max_n = std::max(max_n, probs[i].N);
    launch_k(gemm_finish_kernel, dim3(dim3((M * (max_n / 4) + 255) / 256, n)), dim3(256), 0, st, grp);
  }
  return cudaGetLastError();
}
template <int BN, int FMT>
cudaError_t launch_gemm_wq_t(const GemmMaps &maps, const GemmGroup &grp, dim3 grid, size_t smem, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(gemm_wq_kernel<BN, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  launch_k(gemm_wq_kernel<BN, FMT>, dim3(grid), dim3(WQ_THREADS), smem, st, maps, grp);
  return cudaGetLastError();
}

// shared-memory plan of the packed-weight GEMM inside `avail` bytes: ne buffers (expanded weights + X slot, released
// together) and nw weight slots of `wbox`-byte rows; the weight ring grows first
struct WqPlan { int ne, nw; uint32_t wbox; bool ok; };
WqPlan wq_plan(long long avail, long long buf_bytes, uint32_t wbox, int want_ne, int want_nw) {
  WqPlan p{2, 2, wbox, false};
  const long long ws = (long long)GBM * wbox;
  if (avail - 2 * buf_bytes - 2 * ws < 0) return p;
  p.ok = true;
  for (bool grown = true; grown;) {
    grown = false;
    const long long left = avail - p.ne * buf_bytes - p.nw * ws;
    if (p.nw < want_nw && left >= ws) { ++p.nw; grown = true; continue; }
    if (p.ne < want_ne && left >= buf_bytes) { ++p.ne; grown = true; }
  }
  return p;
}

// quantised weights in packed form (GemmArgs::Wq): any number of rows, walked in tiles of up to 256 along grid.y
cudaError_t launch_gemm_wq(const GemmArgs *probs, int n, cudaStream_t st, int *defer_split) {
  const int M = probs[0].M, fmt = probs[0].wfmt;
  if (fmt != FMT_INT8 && fmt != FMT_INT4) return cudaErrorInvalidValue;
  const int bn = M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  GemmMaps maps;
  GemmGroup grp;
  memset(&grp, 0, sizeof(grp));
  grp.n = n;
  int tiles = 0, min_k1 = 1 << 30;
  bool raw_ok = M <= GEMM_SMALL_M;
  for (int i = 0; i < n; ++i) {
    const GemmArgs &g = probs[i];
    if (g.K % GBK != 0 || g.M < 1 || g.N < 1 || g.M != M || !g.Wq || g.wfmt != fmt) return cudaErrorInvalidValue;
    if (fmt == FMT_INT4 && !g.wq_scale) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.Wq) & 15) || (reinterpret_cast<uintptr_t>(g.A2) & 15))
      return cudaErrorInvalidValue;
    grp.p[i] = g;
    grp.tile_start[i] = tiles;
    tiles += (g.N + GBM - 1) / GBM;
    min_k1 = std::min(min_k1, g.K / GBK);
    raw_ok = raw_ok && g.raw != nullptr && (g.N & 3) == 0 && (g.ldo & 3) == 0;
    if (g.A2) grp.dual |= 1;
  }
  grp.tile_start[n] = tiles;
  const int m_tiles = (M + bn - 1) / bn;
  grp.split = 1;
  grp.stage_bytes = ((grp.dual & 1) ? 2u : 1u) * (uint32_t)bn * GBK * 2;
  const long long buf_bytes = (long long)(fmt == FMT_INT4 ? 2u : 1u) * G_A_BYTES + grp.stage_bytes;
  const uint32_t row_b = fmt == FMT_INT8 ? GBK : GBK / 2;
  // Two CTAs per SM where two or three buffers and a weight ring fit in half an SM's shared memory (up to 64 rows) --
  // the step is a chain of short GEMMs, and a second CTA (of this kernel or, launched early, of the next) hides the
  // hand-overs between the kernel's roles: a quarter of the step time at 32 rows; else one CTA with everything as
  // deep as fits.  Weight slots are as wide as the plan allows.
  WqPlan pl{};
  bool two_per_sm = false;
  for (uint32_t wb = 128; wb >= row_b && !two_per_sm; wb >>= 1) {
    pl = wq_plan(110ll << 10, buf_bytes, wb, 3, wb == 128 ? 3 : wb == 64 ? 4 : 8);
    two_per_sm = pl.ok;
  }
  if (!two_per_sm) pl = wq_plan(225ll << 10, buf_bytes, 128, WQ_MAX_E, 4);
  if (!pl.ok) return cudaErrorInvalidValue;
  for (int i = 0; i < n; ++i) {
    const GemmArgs &g = probs[i];
    const int row_bytes = fmt == FMT_INT8 ? g.K : g.K / 2;
    if (!make_map(&maps.a[i], g.A, g.M, g.K, bn) || !make_map_bytes(&maps.b[i], g.Wq, g.N, row_bytes, (int)pl.wbox))
      return cudaErrorNotSupported;
    if (!make_map(&maps.a2[i], g.A2 ? g.A2 : g.A, g.M, g.K, bn)) return cudaErrorNotSupported;
    maps.b2[i] = maps.b[i];
  }
  for (int i = n; i < GEMM_GROUP_MAX; ++i) { maps.a[i] = maps.a[0]; maps.a2[i] = maps.a2[0]; maps.b[i] = maps.b[0]; maps.b2[i] = maps.b2[0]; }
  const int slots = (two_per_sm ? 2 : 1) * device_sm_count();
  if (raw_ok) {
    // split-K: the fewest waves of CTAs, each at least two K slices long; a slice costs 1, a wave's start and end 2,
    // a slab in the finishing pass a quarter
    const int ctas = tiles * m_tiles, max_split = std::max(1, std::min(GEMM_SPLIT_MAX, min_k1 / 2));
    float best = 0.f;
    for (int sp = 1; sp <= max_split; ++sp) {
      const int waves = (ctas * sp + slots - 1) / slots;
      const float cost = (float)waves * (float)((min_k1 + sp - 1) / sp + 2) + 0.25f * (float)sp;
      if (sp == 1 || cost < best) { best = cost; grp.split = sp; }
    }
  }
  grp.stages = pl.nw;
  grp.estages = pl.ne;
  grp.wbox = pl.wbox;
  const size_t smem = 1024 + (size_t)pl.ne * buf_bytes + (size_t)pl.nw * GBM * pl.wbox + 1024;
  dim3 grid(tiles, m_tiles, grp.split);
  cudaError_t e = cudaErrorInvalidValue;
#define FRB_WQ(BNV) (fmt == FMT_INT8 ? launch_gemm_wq_t<BNV, FMT_INT8>(maps, grp, grid, smem, st) : launch_gemm_wq_t<BNV, FMT_INT4>(maps, grp, grid, smem, st))
  e = bn == 32 ? FRB_WQ(32) : bn == 64 ? FRB_WQ(64) : bn == 128 ? FRB_WQ(128) : FRB_WQ(256);
#undef FRB_WQ
  if (e != cudaSuccess) return e;
  if (defer_split) *defer_split = grp.split;
  if (grp.split > 1 && !defer_split) {
    int max_n = 0;
    for (int i = 0; i < n; ++i) max_n = std::max(max_n, probs[i].N);
    launch_k(gemm_finish_kernel, dim3(dim3((M * (max_n / 4) + 255) / 256, n)), dim3(256), 0, st, grp);
  }
  return cudaGetLastError();
}
}  // namespace

// defer_split (optional): the caller's next kernel sums the split-K slabs itself (ln_mix_seq_kernel, wkv4_rows_kernel);
// it receives the split that was chosen, 1 meaning that the outputs are already complete.
cudaError_t launch_gemm_group(const GemmArgs *probs, int n, int mt, cudaStream_t st, int *defer_split) {
  if (n < 1 || n > GEMM_GROUP_MAX || (mt != 1 && mt != 2)) return cudaErrorInvalidValue;
  const int M = probs[0].M;
  if (defer_split) *defer_split = 1;
  if (probs[0].Wq) return launch_gemm_wq(probs, n, st, defer_split);
  if (M <= GEMM_SMALL_M && wt_enabled()) return launch_gemm_wt(probs, n, st, defer_split);
  // few rows (batched decode): narrow N tiles and split-K, so that a few hundred CTAs stream the weights
  const bool narrow = M <= GEMM_SMALL_M;
  const int bn = narrow ? 64 : 256;
  GemmMaps maps;
  GemmGroup grp;
  memset(&grp, 0, sizeof(grp));
  grp.n = n;
  int tiles = 0, min_k1 = 1 << 30;
  bool raw_ok = true;
  for (int i = 0; i < n; ++i) {
    const GemmArgs &g = probs[i];
    if (g.K % GBK != 0 || g.M < 1 || g.N < 1 || g.M != M) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.Bt) & 15) || (reinterpret_cast<uintptr_t>(g.A2) & 15))
      return cudaErrorInvalidValue;
    if (!make_map(&maps.a[i], g.A, g.M, g.K, GBM) || !make_map(&maps.b[i], g.Bt, g.N, g.K, bn)) return cudaErrorNotSupported;
    if (!make_map(&maps.a2[i], g.A2 ? g.A2 : g.A, g.M, g.K, GBM)) return cudaErrorNotSupported;
    if (!make_map(&maps.b2[i], g.Bt2 ? g.Bt2 : g.Bt, g.N, g.K, bn)) return cudaErrorNotSupported;
    grp.p[i] = g;
    grp.tile_start[i] = tiles;
    tiles += (g.N + bn - 1) / bn;
    min_k1 = std::min(min_k1, g.K / GBK);
    raw_ok = raw_ok && g.raw != nullptr && (g.N & 3) == 0 && (g.ldo & 3) == 0;
  }
  for (int i = n; i < GEMM_GROUP_MAX; ++i) { maps.a[i] = maps.a[0]; maps.a2[i] = maps.a2[0]; maps.b[i] = maps.b[0]; maps.b2[i] = maps.b2[0]; }
  grp.tile_start[n] = tiles;
  const int m_tiles = (M + mt * GBM - 1) / (mt * GBM);
  grp.split = 1;
  if (narrow && raw_ok) {
    const int want = (2 * device_sm_count() + tiles * m_tiles - 1) / (tiles * m_tiles);    // about two CTAs per SM in total
    grp.split = std::max(1, std::min(std::min(want, GEMM_SPLIT_MAX), min_k1 / 4));   // at least 4 K slices per CTA
  }
  if (mt == 1)
    for (int i = 0; i < n; ++i) grp.dual |= probs[i].A2 != nullptr;
  grp.stage_bytes = (uint32_t)(grp.dual ? 2 : 1) * mt * G_A_BYTES + (uint32_t)bn * GBK * 2;
  grp.stages = (int)std::min<size_t>(4, (192u << 10) / grp.stage_bytes);
  if (narrow) grp.stages = 2;   // short K ranges per CTA: a 2-deep ring leaves room for two CTAs per SM (measured: 15 % faster steps)
  const size_t smem = 1024 + (size_t)grp.stages * grp.stage_bytes + 1024;
  dim3 grid(tiles, m_tiles, grp.split);
  cudaError_t e;
  if (narrow) e = mt == 1 ? launch_gemm_t<1, 64>(maps, grp, grid, smem, st) : launch_gemm_t<2, 64>(maps, grp, grid, smem, st);
  else e = mt == 1 ? launch_gemm_t<1, 256>(maps, grp, grid, smem, st) : launch_gemm_t<2, 256>(maps, grp, grid, smem, st);
  if (e != cudaSuccess) return e;
  if (defer_split) *defer_split = grp.split;
  if (grp.split > 1 && !defer_split) {
    int max_n = 0;
    for (int i = 0; i < n; ++i) max_n = std::max(max_n, probs[i].N);
    launch_k(gemm_finish_kernel, dim3(dim3((M * (max_n / 4) + 255) / 256, n)), dim3(256), 0, st, grp);
  }
  return cudaGetLastError();
}

cudaError_t launch_gemm_f16(const GemmArgs &g, cudaStream_t st) {
  return launch_gemm_group(&g, 1, g.M > GBM ? 2 : 1, st, nullptr);   // no raw scratch: no split-K
}

}  // namespace frb
