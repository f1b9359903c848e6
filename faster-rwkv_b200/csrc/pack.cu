// Load-time kernels: dtype casts, the int8 / int4 quantisers (bit-exact with the CPU definition in
// oracle/rwkv_oracle.c), and the repacking of [in,out] matrices into the streaming tile layout
// described in layout.h.  None of this is on the per-token path.
#include "internal.h"

namespace frb {

namespace {

__global__ void k_f16_to_f32(const __half *src, float *dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __half2float(src[i]);
}
__global__ void k_f32_to_f16(const float *src, __half *dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2half_rn(src[i]);
}

// round half away from zero (std::lround semantics); x - trunc(x) is exact in fp32
__device__ __forceinline__ int round_half_away(float x) {
  float t = truncf(x);
  if (fabsf(x - t) >= 0.5f) t += x < 0.f ? -1.f : 1.f;
  return (int)t;
}
// fp16(amax / qmax); 1 when that is zero (all-zero block or underflow) or not finite
__device__ __forceinline__ __half block_scale(float amax, float qmax) {
  __half s = __float2half_rn(amax / qmax);
  unsigned short b = __half_as_ushort(s);
  if ((b & 0x7fffu) == 0 || (b & 0x7c00u) == 0x7c00u) s = __ushort_as_half(0x3c00u);
  return s;
}

// one thread per output channel n: column maximum over k
__global__ void k_scale_int8(const float *W, int K, int N, __half *scales) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float amax = 0.f;
  for (int k = 0; k < K; ++k) amax = fmaxf(amax, fabsf(W[(size_t)k * N + n]));
  scales[n] = block_scale(amax, 127.f);
}
__global__ void k_quant_int8(const float *W, int K, int N, const __half *scales, int8_t *q) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)K * N) return;
  int n = (int)(i / K), k = (int)(i % K);
  float s = __half2float(scales[n]);
  int v = round_half_away(W[(size_t)k * N + n] / s);
  v = v > 127 ? 127 : v < -127 ? -127 : v;
  q[i] = (int8_t)v;
}
// one thread per (n, group of 32 inputs)
__global__ void k_quant_int4(const float *W, int K, int N, uint8_t *packed, __half *scales) {
  const int G = K / 32;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * G) return;
  // consecutive threads take consecutive n so the strided reads of W coalesce
  int n = (int)(i % N), g = (int)(i / N);
  float amax = 0.f;
  for (int k = g * 32; k < g * 32 + 32; ++k) amax = fmaxf(amax, fabsf(W[(size_t)k * N + n]));
  __half sh = block_scale(amax, 7.f);
  float s = __half2float(sh);
  scales[(size_t)n * G + g] = sh;
  for (int k = g * 32; k < g * 32 + 32; k += 2) {
    int v0 = round_half_away(W[(size_t)k * N + n] / s), v1 = round_half_away(W[(size_t)(k + 1) * N + n] / s);
    v0 = v0 > 7 ? 7 : v0 < -7 ? -7 : v0;
    v1 = v1 > 7 ? 7 : v1 < -7 ? -7 : v1;
    packed[(size_t)n * (K / 2) + k / 2] = (uint8_t)((v0 + 8) | ((v1 + 8) << 4));
  }
}
__global__ void k_dequant_int8(const int8_t *q, const __half *scales, int K, int N, float *W) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)K * N) return;
  int k = (int)(i / N), n = (int)(i % N);
  W[i] = (float)q[(size_t)n * K + k] * __half2float(scales[n]);
}
__global__ void k_dequant_int4(const uint8_t *packed, const __half *scales, int K, int N, float *W) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)K * N) return;
  int k = (int)(i / N), n = (int)(i % N);
  uint8_t b = packed[(size_t)n * (K / 2) + k / 2];
  int qv = (int)((k & 1) ? (b >> 4) : (b & 15)) - 8;
  W[i] = (float)qv * __half2float(scales[(size_t)n * (K / 32) + k / 32]);
}

// ---- tile packing ---------------------------------------------------------------------------------

// byte offset of chunk c's weights inside a row block, and of its int4 scales
__device__ __forceinline__ size_t chunk_off(int fmt, int c) {
  if (fmt != FMT_INT4) return (size_t)c * chunk_weight_bytes(fmt);
  const int cps = kt_max(fmt) / CHUNK_K;           // chunks per full stage
  const int s = c / cps, ci = c - s * cps;
  return (size_t)s * stage_bytes(fmt, kt_max(fmt)) + (size_t)ci * 512;
}
__device__ __forceinline__ size_t scale_off_int4(int c, int K) {
  const int cps = kt_max(FMT_INT4) / CHUNK_K;
  const int s = c / cps, ci = c - s * cps;
  const int nch_total = K / CHUNK_K;
  const int nch = min(cps, nch_total - s * cps);   // chunks in this stage
  return (size_t)s * stage_bytes(FMT_INT4, kt_max(FMT_INT4)) + (size_t)nch * 512 + (size_t)ci * 64;
}

// stored code of element (k, n): fp16 bits, int8 + 128, or int4 + 8 (already offset in the source)
__device__ __forceinline__ unsigned code_at(int fmt, const void *src, int K, int N, int k, int n) {
  if (n >= N) return fmt == FMT_FP16 ? 0u : fmt == FMT_INT8 ? 128u : 8u;
  if (fmt == FMT_FP16) return __half_as_ushort(((const __half *)src)[(size_t)k * N + n]);
  if (fmt == FMT_INT8) return (unsigned)(((const int8_t *)src)[(size_t)n * K + k] + 128);
  uint8_t b = ((const uint8_t *)src)[(size_t)n * (K / 2) + k / 2];
  return (k & 1) ? (b >> 4) : (b & 15);
}

// one thread per (row block, chunk, lane)
__global__ void k_pack(int fmt, const void *src, const __half *scales, int K, int N, uint8_t *dst, size_t item_stride,
                       __half *rscale_dst, size_t rscale_stride) {
  const int nch = K / CHUNK_K, nrb = (N + ROWS - 1) / ROWS;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)nrb * nch * 32) return;
  const int lane = (int)(i & 31), c = (int)((i >> 5) % nch), rb = (int)((i >> 5) / nch);
  const int g = lane >> 2, q = lane & 3;
  const int r0 = rb * ROWS + g, r1 = r0 + 8;
  uint8_t *tile = dst + (size_t)rb * item_stride + chunk_off(fmt, c);
  uint32_t words[16];
  for (int j = 0; j < 4; ++j) {
    const int k0 = c * 64 + j * 16 + q * 4;
    unsigned e[8];  // order: (r0,k0) (r0,k0+1) (r1,k0) (r1,k0+1) (r0,k0+2) (r0,k0+3) (r1,k0+2) (r1,k0+3)
    e[0] = code_at(fmt, src, K, N, k0, r0);     e[1] = code_at(fmt, src, K, N, k0 + 1, r0);
    e[2] = code_at(fmt, src, K, N, k0, r1);     e[3] = code_at(fmt, src, K, N, k0 + 1, r1);
    e[4] = code_at(fmt, src, K, N, k0 + 2, r0); e[5] = code_at(fmt, src, K, N, k0 + 3, r0);
    e[6] = code_at(fmt, src, K, N, k0 + 2, r1); e[7] = code_at(fmt, src, K, N, k0 + 3, r1);
    if (fmt == FMT_FP16) {
      for (int t = 0; t < 4; ++t) words[j * 4 + t] = e[2 * t] | (e[2 * t + 1] << 16);
    } else if (fmt == FMT_INT8) {
      words[j * 2 + 0] = e[0] | (e[1] << 8) | (e[2] << 16) | (e[3] << 24);
      words[j * 2 + 1] = e[4] | (e[5] << 8) | (e[6] << 16) | (e[7] << 24);
    } else {
      // nibbles 0..7 = (r0,k0) (r1,k0) (r0,k0+2) (r1,k0+2) (r0,k0+1) (r1,k0+1) (r0,k0+3) (r1,k0+3)
      words[j] = e[0] | (e[2] << 4) | (e[4] << 8) | (e[6] << 12) | (e[1] << 16) | (e[3] << 20) | (e[5] << 24) |
                 (e[7] << 28);
    }
  }
  if (fmt == FMT_FP16) {
    for (int j = 0; j < 4; ++j)
      ((uint4 *)tile)[j * 32 + lane] = make_uint4(words[j * 4], words[j * 4 + 1], words[j * 4 + 2], words[j * 4 + 3]);
  } else if (fmt == FMT_INT8) {
    for (int jj = 0; jj < 2; ++jj)
      ((uint4 *)tile)[jj * 32 + lane] =
          make_uint4(words[jj * 4], words[jj * 4 + 1], words[jj * 4 + 2], words[jj * 4 + 3]);
  } else {
    ((uint4 *)tile)[lane] = make_uint4(words[0], words[1], words[2], words[3]);
    if (q == 0) {
      // group scales of this chunk for rows g and g+8
      __half *sc = (__half *)(dst + (size_t)rb * item_stride + scale_off_int4(c, K)) + g * 4;
      const int G = K / 32;
      const __half zero = __ushort_as_half(0);
      sc[0] = r0 < N ? scales[(size_t)r0 * G + c * 2] : zero;
      sc[1] = r1 < N ? scales[(size_t)r1 * G + c * 2] : zero;
      sc[2] = r0 < N ? scales[(size_t)r0 * G + c * 2 + 1] : zero;
      sc[3] = r1 < N ? scales[(size_t)r1 * G + c * 2 + 1] : zero;
    }
  }
  if (fmt == FMT_INT8 && c == 0 && q == 0 && rscale_dst) {
    const __half zero = __ushort_as_half(0);
    rscale_dst[(size_t)rb * rscale_stride + g] = r0 < N ? scales[r0] : zero;
    rscale_dst[(size_t)rb * rscale_stride + g + 8] = r1 < N ? scales[r1] : zero;
  }
}

// one thread per element (k, n): read it back out of the tiles, dequantised
__global__ void k_unpack(int fmt, const uint8_t *tiles, size_t item_stride, const __half *rscale, size_t rscale_stride,
                         int K, int N, float *W) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)K * N) return;
  const int k = (int)(i / N), n = (int)(i % N);
  const int rb = n / ROWS, r = n % ROWS, g = r & 7, hi = r >> 3;
  const int c = k >> 6, j = (k >> 4) & 3, q = (k >> 2) & 3, s = k & 3;
  const int lane = g * 4 + q;
  const uint8_t *tile = tiles + (size_t)rb * item_stride + chunk_off(fmt, c);
  const int idx = (s >> 1) * 4 + hi * 2 + (s & 1);  // position among the 8 elements of (lane, j)
  float v;
  if (fmt == FMT_FP16) {
    v = __half2float(((const __half *)(tile + ((size_t)j * 32 + lane) * 16))[idx]);
  } else if (fmt == FMT_INT8) {
    int code = (tile + ((size_t)(j >> 1) * 32 + lane) * 16)[(j & 1) * 8 + idx];
    v = (float)(code - 128) * __half2float(rscale[(size_t)rb * rscale_stride + r]);
  } else {
    uint32_t w = ((const uint32_t *)(tile + (size_t)lane * 16))[j];
    const int nib = ((s & 1) << 2) | ((s >> 1) << 1) | hi;
    int code = (w >> (4 * nib)) & 15;
    const __half *sc = (const __half *)(tiles + (size_t)rb * item_stride + scale_off_int4(c, K)) + g * 4;
    v = (float)(code - 8) * __half2float(sc[((j >> 1) << 1) + hi]);
  }
  W[i] = v;
}

inline unsigned blocks_for(size_t n, int bs) { return (unsigned)((n + bs - 1) / bs); }

}  // namespace

cudaError_t launch_f16_to_f32(const __half *src, float *dst, size_t n, cudaStream_t st) {
  if (n) k_f16_to_f32<<<blocks_for(n, 256), 256, 0, st>>>(src, dst, n);
  return cudaGetLastError();
}
namespace {
__global__ void k_i8_to_f16(const int8_t *src, __half *dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __int2half_rn((int)src[i]);
}
// hi = fp16(x), lo = fp16(x - hi): together they carry ~22 bits of x
__global__ void k_f32_split_f16(const float *src, __half *hi, __half *lo, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const __half h = __float2half_rn(src[i]);
    hi[i] = h;
    lo[i] = __float2half_rn(src[i] - __half2float(h));
  }
}
}  // namespace
cudaError_t launch_i8_to_f16(const int8_t *src, __half *dst, size_t n, cudaStream_t st) {
  if (n) k_i8_to_f16<<<blocks_for(n, 256), 256, 0, st>>>(src, dst, n);
  return cudaGetLastError();
}
cudaError_t launch_f32_split_f16(const float *src, __half *hi, __half *lo, size_t n, cudaStream_t st) {
  if (n) k_f32_split_f16<<<blocks_for(n, 256), 256, 0, st>>>(src, hi, lo, n);
  return cudaGetLastError();
}
cudaError_t launch_f32_to_f16(const float *src, __half *dst, size_t n, cudaStream_t st) {
  if (n) k_f32_to_f16<<<blocks_for(n, 256), 256, 0, st>>>(src, dst, n);
  return cudaGetLastError();
}
cudaError_t launch_quant_int8(const float *W, int K, int N, int8_t *q, __half *scales, cudaStream_t st) {
  k_scale_int8<<<blocks_for(N, 128), 128, 0, st>>>(W, K, N, scales);
  k_quant_int8<<<blocks_for((size_t)K * N, 256), 256, 0, st>>>(W, K, N, scales, q);
  return cudaGetLastError();
}
cudaError_t launch_quant_int4(const float *W, int K, int N, uint8_t *packed, __half *scales, cudaStream_t st) {
  k_quant_int4<<<blocks_for((size_t)N * (K / 32), 128), 128, 0, st>>>(W, K, N, packed, scales);
  return cudaGetLastError();
}
cudaError_t launch_dequant_int8(const int8_t *q, const __half *scales, int K, int N, float *W, cudaStream_t st) {
  k_dequant_int8<<<blocks_for((size_t)K * N, 256), 256, 0, st>>>(q, scales, K, N, W);
  return cudaGetLastError();
}
cudaError_t launch_dequant_int4(const uint8_t *packed, const __half *scales, int K, int N, float *W, cudaStream_t st) {
  k_dequant_int4<<<blocks_for((size_t)K * N, 256), 256, 0, st>>>(packed, scales, K, N, W);
  return cudaGetLastError();
}
cudaError_t launch_pack(int fmt, const void *src, const __half *scales, int K, int N, uint8_t *dst, size_t item_stride,
                        __half *rscale_dst, size_t rscale_stride, cudaStream_t st) {
  const size_t n = (size_t)((N + ROWS - 1) / ROWS) * (K / CHUNK_K) * 32;
  k_pack<<<blocks_for(n, 128), 128, 0, st>>>(fmt, src, scales, K, N, dst, item_stride, rscale_dst, rscale_stride);
  return cudaGetLastError();
}
cudaError_t launch_unpack(int fmt, const uint8_t *tiles, size_t item_stride, const __half *rscale, size_t rscale_stride,
                          int K, int N, float *W, cudaStream_t st) {
  k_unpack<<<blocks_for((size_t)K * N, 256), 256, 0, st>>>(fmt, tiles, item_stride, rscale, rscale_stride, K, N, W);
  return cudaGetLastError();
}

}  // namespace frb
