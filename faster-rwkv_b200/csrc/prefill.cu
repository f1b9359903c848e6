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

#include <cstdint>

#include "common.cuh"
#include "internal.h"

namespace frb {

namespace {

// ------------------------------------------------------------------------------------------------
// tcgen05 GEMM: out[M, N] = epilogue(A[M, K] . Bt[N, K]^T), fp16 operands (both K-major), fp32 accumulate.
// One CTA per 128 x 256 output tile; K is walked in 64-wide slices through a 4-deep TMA ring.
//   warp 0 (one lane): TMA producer          warp 1 (one lane): MMA issue; the warp owns the TMEM allocation
//   warps 2..5: epilogue, one TMEM lane quadrant (32 rows) each
constexpr int GBM = 128, GBN = 256, GBK = 64, GSTAGES = 4;
constexpr int G_THREADS = 192;
constexpr uint32_t G_A_BYTES = GBM * GBK * 2, G_B_BYTES = GBN * GBK * 2, G_STAGE_BYTES = G_A_BYTES + G_B_BYTES;
constexpr size_t G_SMEM = 1024 /* barriers */ + (size_t)GSTAGES * G_STAGE_BYTES + 1024 /* alignment slack */;
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
constexpr uint32_t G_IDESC = (1u << 4) | ((uint32_t)(GBN >> 3) << 17) | ((uint32_t)(GBM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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

__device__ __forceinline__ float sigmoid_g(float v) { return 1.f / (1.f + expf(-v)); }

// Epilogue of 32 consecutive columns of one output row.
__device__ __forceinline__ void gemm_epilogue_row(const GemmArgs &g, int row, int col0, const uint32_t (&acc)[32]) {
  const int ncol = min(32, g.N - col0);
  if (ncol <= 0) return;
  const size_t o = (size_t)row * g.ldo + col0;
  if (g.epi == GEMM_EPI_F32) {
    float *out = reinterpret_cast<float *>(g.out) + o;
    if (ncol == 32) {
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
    for (int i = 0; i < ncol; ++i) {
      float a = __uint_as_float(acc[i]);
      if (g.epi == GEMM_EPI_MULADD_F32) a *= __half2float(r[i]);
      out[i] = (x[i] + a) * g.scale;
    }
    return;
  }
  __half *out = reinterpret_cast<__half *>(g.out) + o;
  for (int i = 0; i < ncol; i += 2) {
    float a = __uint_as_float(acc[i]), b = i + 1 < ncol ? __uint_as_float(acc[i + 1]) : 0.f;
    if (g.epi == GEMM_EPI_SILU_F16) { a = a * sigmoid_g(a); b = b * sigmoid_g(b); }
    else if (g.epi == GEMM_EPI_SIGMOID_F16) { a = sigmoid_g(a); b = sigmoid_g(b); }
    else if (g.epi == GEMM_EPI_RELU2_F16) { a = fmaxf(a, 0.f); a *= a; b = fmaxf(b, 0.f); b *= b; }
    if (i + 1 < ncol) *reinterpret_cast<__half2 *>(out + i) = __floats2half2_rn(a, b);
    else out[i] = __float2half_rn(a);
  }
}

__global__ void __launch_bounds__(G_THREADS, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmArgs g) {
  extern __shared__ uint8_t gsm_raw[];
  // barriers in the first KB, tiles from the next 1024-byte boundary
  uint8_t *gsm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *full = reinterpret_cast<uint64_t *>(gsm);
  uint64_t *empty = full + GSTAGES;
  uint64_t *acc_full = empty + GSTAGES;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  const uint32_t tiles = smem_u32(gsm + 1024);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_m = blockIdx.y, tile_n = blockIdx.x;
  const int num_k = g.K / GBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)GBN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % GSTAGES;
        const uint32_t parity = ((kb / GSTAGES) & 1) ^ 1;   // a fresh barrier reads as "previous phase complete"
        if (!mbar_wait(&empty[s], parity, abort_flag, g.status, ST_GEMM_TIMEOUT)) break;
        mbar_expect_tx(&full[s], G_STAGE_BYTES);
        const uint32_t a_dst = tiles + (uint32_t)s * G_STAGE_BYTES;
        tma_load_2d(a_dst, &tma_a, kb * GBK, tile_m * GBM, &full[s]);
        tma_load_2d(a_dst + G_A_BYTES, &tma_b, kb * GBK, tile_n * GBN, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool live = true;
      for (int kb = 0; kb < num_k && live; ++kb) {
        const int s = kb % GSTAGES;
        if (!mbar_wait(&full[s], (kb / GSTAGES) & 1, abort_flag, g.status, ST_GEMM_TIMEOUT)) { live = false; break; }
        tc_fence_after();
        const uint32_t a_addr = tiles + (uint32_t)s * G_STAGE_BYTES;
        const uint64_t ad = umma_desc_k128(a_addr), bd = umma_desc_k128(a_addr + G_A_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < GBK / 16; ++k4)   // 16 inputs = 32 bytes further along the swizzled rows
          umma_f16(tmem_base, ad + (uint64_t)(k4 * 2), bd + (uint64_t)(k4 * 2), G_IDESC, (kb | k4) != 0);
        umma_commit(&empty[s]);   // the slot is free once these MMAs have read it
      }
      umma_commit(acc_full);      // the accumulator is complete once every MMA has retired
    }
  } else {
    // epilogue warps 2..5 -> TMEM lane quadrants 2, 3, 0, 1
    const int quad = warp & 3;
    const bool ok = mbar_wait(acc_full, 0, abort_flag, g.status, ST_GEMM_TIMEOUT);
    tc_fence_after();
    const int row = tile_m * GBM + quad * 32 + lane;
    if (ok) {
      for (int c0 = 0; c0 < GBN; c0 += 32) {
        if (tile_n * GBN + c0 >= g.N) break;   // warp-uniform
        uint32_t acc[32];
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, acc);
        if (row < g.M) gemm_epilogue_row(g, row, tile_n * GBN + c0, acc);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)GBN) : "memory");
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

cudaError_t launch_gemm_f16(const GemmArgs &g, cudaStream_t st) {
  if (g.K % GBK != 0 || g.M < 1 || g.N < 1) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.Bt) & 15)) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!make_map(&ma, g.A, g.M, g.K, GBM) || !make_map(&mb, g.Bt, g.N, g.K, GBN)) return cudaErrorNotSupported;
  cudaError_t e = cudaFuncSetAttribute(gemm_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G_SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid((g.N + GBN - 1) / GBN, (g.M + GBM - 1) / GBM);
  gemm_f16_kernel<<<grid, G_THREADS, G_SMEM, st>>>(ma, mb, g);
  return cudaGetLastError();
}

}  // namespace frb
