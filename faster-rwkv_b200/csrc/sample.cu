// Sampling on the device: Sampler::Sample (sampler.cpp:38-101) without copying the [V] logits to the host and
// without the host's std::sort over V entries per token.
//   probs = softmax(logits)   (kernels/cpu/softmax.cpp:6-21, temperature 1)
//   sort descending; keep the shortest prefix whose cumulative probability reaches top_p; cut to top_k if top_k > 0;
//   weights = probs ^ (1 / clamp(temperature, 0.1, 5)); draw the first index whose running sum reaches u * total.
// The uniform draw u in [0, 1] comes from the caller (the reference takes (g() - min) / (max - min) of a
// std::minstd_rand0, sampler.cpp:20-22), so a host that seeds the same generator reproduces the reference's picks.
#include <cuda_runtime.h>

#include <cub/device/device_segmented_radix_sort.cuh>

#include <cstdint>

#include "internal.h"

namespace frb {

namespace {

// probs[row][i] = exp(l_i - max) / sum, ids[row][i] = i; one CTA per row
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float *logits, int V, int ld, float *probs, int32_t *ids) {
  __shared__ float red[8];
  __shared__ float bc;
  const float *row = logits + (size_t)blockIdx.x * ld;
  float *p = probs + (size_t)blockIdx.x * V;
  int32_t *id = ids + (size_t)blockIdx.x * V;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) { float m = red[0]; for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]); bc = m; }
  __syncthreads();
  mx = bc;
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) { const float e = expf(row[i] - mx); p[i] = e; s += e; }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) { float t = 0.f; for (int w = 0; w < 8; ++w) t += red[w]; bc = t; }
  __syncthreads();
  const float inv = 1.f / bc;
  for (int i = threadIdx.x; i < V; i += blockDim.x) { p[i] *= inv; id[i] = i; }
}

__global__ void segment_offsets_kernel(int rows, int V, int *off) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i <= rows) off[i] = i * V;
}

// Block-wide exclusive prefix sum of one value per thread (256 threads); total = the sum over the block.
__device__ __forceinline__ float block_excl_scan(float v, float *sh, float &total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();                 // sh may still be read from the previous call
  if (lane == 31) sh[warp] = inc;
  __syncthreads();
  float base = 0.f, tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    if (w < warp) base += sh[w];
    tot += sh[w];
  }
  total = tot;
  return base + inc - v;
}

// One CTA per row over the sorted probabilities: the reference's three loops (top-p prefix, temperature weights, the
// inverse-CDF walk: sampler.cpp:59-66, 86-93, 22-30) each become a per-thread walk over a contiguous segment plus a
// block scan of the segment sums.  Running sums therefore differ from the reference's strictly serial ones by fp32
// rounding only; a draw that lands within that distance of a threshold may resolve to the neighbouring entry.
__global__ void __launch_bounds__(256) pick_rows_kernel(const float *sorted_p, const int32_t *sorted_id, int V, float temperature, int top_k,
                                                        float top_p, const float *u, int32_t *out) {
  __shared__ float sh[8];
  __shared__ int cut;
  const int row = blockIdx.x;
  const float *p = sorted_p + (size_t)row * V;
  const int S = (V + 255) / 256, lo = min(V, (int)threadIdx.x * S), hi = min(V, lo + S);
  if (threadIdx.x == 0) cut = V;
  // top-p: the shortest prefix whose running sum reaches top_p
  float seg = 0.f, total;
  for (int i = lo; i < hi; ++i) seg += p[i];
  float before = block_excl_scan(seg, sh, total);
  if (before < top_p && before + seg >= top_p) {
    float c = before;
    for (int i = lo; i < hi; ++i) {
      c += p[i];
      if (c >= top_p) { atomicMin(&cut, i + 1); break; }
    }
  }
  __syncthreads();
  int len = cut;
  if (top_k > 0) len = min(len, top_k);
  __syncthreads();
  // weights p ^ (1 / temperature) over the kept prefix, then the first entry whose running weight reaches u * total
  const float it = 1.f / fminf(fmaxf(temperature, 0.1f), 5.f);
  const int h2 = min(hi, len);
  seg = 0.f;
  for (int i = lo; i < h2; ++i) seg += powf(p[i], it);
  before = block_excl_scan(seg, sh, total);
  const float rv = u[row] * total;
  if (threadIdx.x == 0) cut = len - 1;
  __syncthreads();
  if (lo < h2 && before < rv && before + seg >= rv) {
    float c = before;
    for (int i = lo; i < h2; ++i) {
      c += powf(p[i], it);
      if (c >= rv) { atomicMin(&cut, i); break; }
    }
  }
  if (threadIdx.x == 0 && rv <= 0.f) atomicMin(&cut, 0);   // u = 0: the first entry already reaches the draw
  __syncthreads();
  if (threadIdx.x == 0) out[row] = sorted_id[(size_t)row * V + cut];
}

// logits[stream[i]][token[i]] += delta[i]: the sparse adjustments a chat loop makes before sampling (frequency /
// presence penalties and the end-of-text / newline biases of chat.cpp:57-75), without the logits leaving the device
__global__ void logits_add_kernel(float *logits, int ld, const int32_t *stream, const int32_t *token, const float *delta, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) atomicAdd(logits + (size_t)stream[i] * ld + token[i], delta[i]);
}

}  // namespace

size_t sample_scratch_bytes(int rows, int V) {
  size_t temp = 0;
  cub::DeviceSegmentedRadixSort::SortPairsDescending(nullptr, temp, (const float *)nullptr, (float *)nullptr, (const int32_t *)nullptr,
                                                     (int32_t *)nullptr, rows * V, rows, (const int *)nullptr, (const int *)nullptr);
  const size_t n = (size_t)rows * V;
  return 4 * n * 4 + ((size_t)rows + 1) * 4 + 256 + temp + 256;
}

// scratch: sample_scratch_bytes(rows, V) bytes; u: device [rows]; out: device [rows]
cudaError_t launch_sample_rows(const float *logits, int rows, int V, int ld, float temperature, int top_k, float top_p,
                               const float *u, int32_t *out, void *scratch, size_t scratch_bytes, cudaStream_t st) {
  const size_t n = (size_t)rows * V;
  float *probs = reinterpret_cast<float *>(scratch), *sorted_p = probs + n;
  int32_t *ids = reinterpret_cast<int32_t *>(sorted_p + n), *sorted_id = ids + n;
  int *off = reinterpret_cast<int *>(sorted_id + n);
  uint8_t *temp = reinterpret_cast<uint8_t *>(off) + (((size_t)rows + 1) * 4 + 255) / 256 * 256;
  size_t temp_bytes = scratch_bytes - (size_t)(temp - reinterpret_cast<uint8_t *>(scratch));
  softmax_rows_kernel<<<rows, 256, 0, st>>>(logits, V, ld, probs, ids);
  segment_offsets_kernel<<<(rows + 256) / 256, 256, 0, st>>>(rows, V, off);
  cudaError_t e = cub::DeviceSegmentedRadixSort::SortPairsDescending(temp, temp_bytes, probs, sorted_p, ids, sorted_id, (int)n, rows, off,
                                                                     off + 1, 0, 32, st);
  if (e != cudaSuccess) return e;
  pick_rows_kernel<<<rows, 256, 0, st>>>(sorted_p, sorted_id, V, temperature, top_k, top_p, u, out);
  return cudaGetLastError();
}

cudaError_t launch_logits_add(float *logits, int ld, const int32_t *stream, const int32_t *token, const float *delta, int n, cudaStream_t st) {
  if (n > 0) logits_add_kernel<<<(n + 255) / 256, 256, 0, st>>>(logits, ld, stream, token, delta, n);
  return cudaGetLastError();
}

}  // namespace frb
