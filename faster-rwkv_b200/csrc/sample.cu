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

// one thread per row walks the sorted probabilities in order, exactly as the reference's loops do
__global__ void pick_rows_kernel(const float *sorted_p, const int32_t *sorted_id, int V, float temperature, int top_k, float top_p,
                                 const float *u, int32_t *out, int rows) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const float *p = sorted_p + (size_t)row * V;
  int len = V;
  float cum = 0.f;
  for (int i = 0; i < V; ++i) {
    cum += p[i];
    if (cum >= top_p) { len = i + 1; break; }
  }
  if (top_k > 0) len = min(len, top_k);
  const float it = 1.f / fminf(fmaxf(temperature, 0.1f), 5.f);
  float total = 0.f;
  for (int i = 0; i < len; ++i) total += powf(p[i], it);
  const float rv = u[row] * total;
  cum = 0.f;
  int pick = len - 1;
  for (int i = 0; i < len; ++i) {
    cum += powf(p[i], it);
    if (cum >= rv) { pick = i; break; }
  }
  out[row] = sorted_id[(size_t)row * V + pick];
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
  pick_rows_kernel<<<(rows + 63) / 64, 64, 0, st>>>(sorted_p, sorted_id, V, temperature, top_k, top_p, u, out, rows);
  return cudaGetLastError();
}

}  // namespace frb
