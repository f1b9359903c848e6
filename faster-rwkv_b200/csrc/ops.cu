// Stand-alone operators over plain device pointers: the pieces of the forward pass as the reference's operator API
// cuts them (kernels/kernels.h:15-257), for its op-grained call path (def::ModelForward calling att / ffn /
// layernorm / matmul per op, kernels/default/model_forward.cpp:105-188) and for per-kernel parity tests.  The
// persistent decode kernel and the seq path fuse all of this; these entry points exist so that each formula can be
// checked, and registered, on its own.  Nothing here is on the fast path.
#include <cstring>
#include <string>

#include "../../include/fr_b200.h"
#include "internal.h"

using namespace frb;

namespace {

thread_local std::string g_op_err;
int op_fail(int code, const std::string &msg) { g_op_err = msg; return code; }
#define OP_CU(call)                                                                                          \
  do {                                                                                                       \
    cudaError_t e_ = (call);                                                                                 \
    if (e_ != cudaSuccess) return op_fail(FR_B200_E_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
  } while (0)

__device__ __forceinline__ float ldv(const void *p, size_t i, int dt) {
  return dt == FR_B200_T_F16 ? __half2float(reinterpret_cast<const __half *>(p)[i]) : reinterpret_cast<const float *>(p)[i];
}
__device__ __forceinline__ void stv(void *p, size_t i, int dt, float v) {
  if (dt == FR_B200_T_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
  else reinterpret_cast<float *>(p)[i] = v;
}
__device__ __forceinline__ float sigmoid_op(float v) { return 1.f / (1.f + expf(-v)); }

// block-wide sum of two values (blockDim.x = 256)
__device__ __forceinline__ float2 block_sum2_op(float a, float b, float *red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, o);
    b += __shfl_xor_sync(0xffffffffu, b, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) { red[warp * 2] = a; red[warp * 2 + 1] = b; }
  __syncthreads();
  float sa = 0.f, sb = 0.f;
  for (int w = 0; w < 8; ++w) { sa += red[w * 2]; sb += red[w * 2 + 1]; }
  return make_float2(sa, sb);
}

// LayerNorm of every row (layer_norm.cu:101-130: fp32 statistics, eps 1e-5) and, with nvec > 0, the token-shift mix
// of att.cu:90-143 / ffn.cu:15-32: out_v = xx * mix_v + sx * (1 - mix_v).  One CTA per row.
struct LnMixOp {
  const void *x, *sx, *w, *b, *mix[4];
  void *xx, *out[4];
  int C, nvec, x_dt, p_dt, o_dt;   // dtypes of x / sx / xx, of the parameters, of the mixed outputs
};
__global__ void __launch_bounds__(256) ln_mix_op_kernel(LnMixOp a) {
  __shared__ float red[16];
  const size_t row = (size_t)blockIdx.x * a.C;
  float s1 = 0.f, s2 = 0.f;
  const float piv = ldv(a.x, row, a.x_dt);
  for (int i = threadIdx.x; i < a.C; i += blockDim.x) {
    const float d = ldv(a.x, row + i, a.x_dt) - piv;
    s1 += d; s2 += d * d;
  }
  const float2 s = block_sum2_op(s1, s2, red);
  const float m = s.x / (float)a.C;
  float var = s.y / (float)a.C - m * m;
  var = var > 0.f ? var : 0.f;
  const float mean = piv + m, rstd = rsqrtf(var + 1e-5f);
  for (int i = threadIdx.x; i < a.C; i += blockDim.x) {
    const float xn = (ldv(a.x, row + i, a.x_dt) - mean) * rstd * ldv(a.w, i, a.p_dt) + ldv(a.b, i, a.p_dt);
    if (a.xx) stv(a.xx, row + i, a.x_dt, xn);
    if (a.nvec > 0) {
      const float sxv = ldv(a.sx, row + i, a.x_dt);
      for (int v = 0; v < a.nvec; ++v) {
        const float mv = ldv(a.mix[v], i, a.p_dt);
        stv(a.out[v], row + i, a.o_dt, xn * mv + sxv * (1.f - mv));
      }
    }
  }
}

// WkvForwardOne (att.cu:30-62) with the sigmoid of att.cu:154-159: one thread per channel, new state tensors
struct Wkv4Op {
  const float *k, *v, *r, *decay, *first, *aa, *bb, *pp;
  float *aa2, *bb2, *pp2;
  void *out;
  int C, o_dt;
};
__global__ void __launch_bounds__(256) wkv4_step_kernel(Wkv4Op a) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= a.C) return;
  const float k = a.k[c], v = a.v[c], r = sigmoid_op(a.r[c]);
  const float aa = a.aa[c], bb = a.bb[c], pp = a.pp[c], u = a.first[c], w = a.decay[c];
  float ww = u + k;
  float pm = fmaxf(pp, ww);
  float e1 = expf(pp - pm), e2 = expf(ww - pm);
  stv(a.out, c, a.o_dt, r * ((e1 * aa + e2 * v) / (e1 * bb + e2)));
  ww = w + pp;
  pm = fmaxf(ww, k);
  e1 = expf(ww - pm);
  e2 = expf(k - pm);
  a.aa2[c] = e1 * aa + e2 * v;
  a.bb2[c] = e1 * bb + e2;
  a.pp2[c] = pm;
}

// OneV5MulAdd + the readout matmul of _ATT_ONE_V5 / _ATT_ONE_V5_1 (att.cu:64-81, 219-335): per head
//   y[j] = sum_i r[i] * (u_i * k[i] * v[j] + s[i][j]),   s'[i][j] = w_i * s[i][j] + k[i] * v[j]
// one CTA per head, thread j owns value column j (coalesced over j); decay / first per head (5.0) or per (head, i)
__global__ void __launch_bounds__(64) wkv5_step_kernel(const float *r, const float *k, const float *v, const float *decay,
                                                       const float *first, const float *s, float *s2, float *y, int per_head) {
  const int h = blockIdx.x, j = threadIdx.x;
  const float vj = v[h * 64 + j];
  float acc = 0.f;
  for (int i = 0; i < 64; ++i) {
    const float ki = k[h * 64 + i], ri = r[h * 64 + i];
    const float u = per_head ? first[h] : first[h * 64 + i], w = per_head ? decay[h] : decay[h * 64 + i];
    const float sv = s[((size_t)h * 64 + i) * 64 + j], x = ki * vj;
    acc += ri * (u * x + sv);
    s2[((size_t)h * 64 + i) * 64 + j] = w * sv + x;
  }
  y[h * 64 + j] = acc;
}

// GroupNorm over the last dimension cut into num_groups pieces (group_norm.cu:322-357): one warp per (row, group)
__global__ void __launch_bounds__(256) groupnorm_op_kernel(const void *x, const void *w, const void *b, void *out, int rows, int C,
                                                           int groups, int x_dt, int p_dt) {
  const int unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (unit >= rows * groups) return;
  const int row = unit / groups, gi = unit - row * groups, gs = C / groups;
  const size_t base = (size_t)row * C + (size_t)gi * gs;
  float s = 0.f;
  for (int i = lane; i < gs; i += 32) s += ldv(x, base + i, x_dt);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float mean = s / (float)gs;
  float q = 0.f;
  for (int i = lane; i < gs; i += 32) { const float d = ldv(x, base + i, x_dt) - mean; q += d * d; }
  for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
  const float rstd = rsqrtf(q / (float)gs + 1e-5f);
  for (int i = lane; i < gs; i += 32) {
    const int c = gi * gs + i;
    stv(out, base + i, x_dt, (ldv(x, base + i, x_dt) - mean) * rstd * ldv(w, c, p_dt) + ldv(b, c, p_dt));
  }
}

// element-wise: out[i] = f(x[i], y[i], z[i]) with per-operand dtypes; the operands may be null where unused
__global__ void __launch_bounds__(256) elementwise_op_kernel(int op, const void *x, int x_dt, const void *y, int y_dt, const void *z,
                                                             int z_dt, float alpha, void *out, int o_dt, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float a = x ? ldv(x, i, x_dt) : 0.f, b = y ? ldv(y, i, y_dt) : 0.f, c = z ? ldv(z, i, z_dt) : 0.f;
  float r;
  switch (op) {
    case FR_B200_EW_COPY: r = a; break;
    case FR_B200_EW_FILL: r = alpha; break;
    case FR_B200_EW_SCALE: r = a * alpha; break;
    case FR_B200_EW_ADD: r = a + b; break;
    case FR_B200_EW_MUL: r = a * b; break;
    case FR_B200_EW_SIGMOID: r = sigmoid_op(a); break;
    case FR_B200_EW_RELU2: { const float t = fmaxf(a, 0.f); r = t * t; break; }
    case FR_B200_EW_SILU: r = a * sigmoid_op(a); break;
    case FR_B200_EW_FMA: r = a * b + c; break;
    default: r = 0.f;
  }
  stv(out, i, o_dt, r);
}

bool bad_dt(int dt) { return dt != FR_B200_T_F16 && dt != FR_B200_T_F32; }

struct OpBuf {
  void *p = nullptr;
  ~OpBuf() { if (p) cudaFree(p); }
  cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 256); }
};

}  // namespace

extern "C" {

const char *fr_b200_op_last_error(void) { return g_op_err.c_str(); }

int fr_b200_ln_mix(const void *x, const void *sx, const void *ln_w, const void *ln_b, const void *const *mix, int nvec, int rows,
                   int C, int act_dtype, int param_dtype, int out_dtype, void *xx, void *const *out, void *stream) {
  if (!x || !ln_w || !ln_b || rows < 1 || C < 1 || nvec < 0 || nvec > 4) return op_fail(FR_B200_E_ARG, "bad argument");
  if (bad_dt(act_dtype) || bad_dt(param_dtype) || bad_dt(out_dtype)) return op_fail(FR_B200_E_ARG, "dtype must be f16 or f32");
  if (nvec > 0 && (!sx || !mix || !out)) return op_fail(FR_B200_E_ARG, "mix needs sx, mix vectors and outputs");
  if (nvec == 0 && !xx) return op_fail(FR_B200_E_ARG, "nothing to write");
  LnMixOp a;
  std::memset(&a, 0, sizeof(a));
  a.x = x; a.sx = sx; a.w = ln_w; a.b = ln_b; a.xx = xx; a.C = C; a.nvec = nvec;
  a.x_dt = act_dtype; a.p_dt = param_dtype; a.o_dt = out_dtype;
  for (int v = 0; v < nvec; ++v) {
    if (!mix[v] || !out[v]) return op_fail(FR_B200_E_ARG, "null mix vector or output");
    a.mix[v] = mix[v]; a.out[v] = out[v];
  }
  ln_mix_op_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  OP_CU(cudaGetLastError());
  return FR_B200_OK;
}

int fr_b200_wkv4_step(const float *k, const float *v, const float *r, const float *decay, const float *first, const float *aa,
                      const float *bb, const float *pp, int C, int out_dtype, void *out, float *aa2, float *bb2, float *pp2,
                      void *stream) {
  if (!k || !v || !r || !decay || !first || !aa || !bb || !pp || !out || !aa2 || !bb2 || !pp2 || C < 1)
    return op_fail(FR_B200_E_ARG, "bad argument");
  if (bad_dt(out_dtype)) return op_fail(FR_B200_E_ARG, "dtype must be f16 or f32");
  Wkv4Op a = {k, v, r, decay, first, aa, bb, pp, aa2, bb2, pp2, out, C, out_dtype};
  wkv4_step_kernel<<<(C + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  OP_CU(cudaGetLastError());
  return FR_B200_OK;
}

int fr_b200_wkv5_step(const float *r, const float *k, const float *v, const float *decay, const float *first, int per_head,
                      const float *s, int n_head, float *s2, float *y, void *stream) {
  if (!r || !k || !v || !decay || !first || !s || !s2 || !y || n_head < 1) return op_fail(FR_B200_E_ARG, "bad argument");
  wkv5_step_kernel<<<n_head, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(r, k, v, decay, first, s, s2, y, per_head);
  OP_CU(cudaGetLastError());
  return FR_B200_OK;
}

int fr_b200_wkv5_chunk_scan(const float *r, const float *k, const float *v, const float *decay, const float *first, int per_head,
                            float *state, int n_head, int T, int n_chunks, float *y, void *stream) {
  if (!r || !k || !v || !decay || !first || !state || !y || n_head < 1 || T < 1 || n_chunks < 1 || n_chunks > T)
    return op_fail(FR_B200_E_ARG, "bad argument");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  SeqWkvArgs a;
  std::memset(&a, 0, sizeof(a));
  a.r = r; a.k = k; a.v = v; a.decay = decay; a.first = first; a.state = state; a.y = y; a.T = T; a.C = n_head * 64;
  a.per_head = per_head;
  a.chunk_len = (T + n_chunks - 1) / n_chunks;
  a.n_chunks = (T + a.chunk_len - 1) / a.chunk_len;
  OpBuf e, sin;
  if (a.n_chunks > 1) {
    OP_CU(e.alloc((size_t)n_head * a.n_chunks * 4096 * 4));
    OP_CU(sin.alloc((size_t)n_head * a.n_chunks * 4096 * 4));
    a.e_out = reinterpret_cast<float *>(e.p); a.s_in = reinterpret_cast<float *>(sin.p);
  }
  OP_CU(launch_wkv5_seq(a, n_head, st));
  OP_CU(cudaStreamSynchronize(st));   // the scratch goes away with this call
  return FR_B200_OK;
}

int fr_b200_groupnorm(const void *x, const void *w, const void *b, int rows, int C, int num_groups, int x_dtype, int param_dtype,
                      void *out, void *stream) {
  if (!x || !w || !b || !out || rows < 1 || C < 1 || num_groups < 1 || C % num_groups) return op_fail(FR_B200_E_ARG, "bad argument");
  if (bad_dt(x_dtype) || bad_dt(param_dtype)) return op_fail(FR_B200_E_ARG, "dtype must be f16 or f32");
  groupnorm_op_kernel<<<(rows * num_groups + 7) / 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x, w, b, out, rows, C,
                                                                                                      num_groups, x_dtype, param_dtype);
  OP_CU(cudaGetLastError());
  return FR_B200_OK;
}

int fr_b200_elementwise(int op, const void *x, int x_dtype, const void *y, int y_dtype, const void *z, int z_dtype, float alpha,
                        void *out, int out_dtype, size_t n, void *stream) {
  if (op < FR_B200_EW_COPY || op > FR_B200_EW_FMA || !out) return op_fail(FR_B200_E_ARG, "bad argument");
  if (bad_dt(out_dtype) || (x && bad_dt(x_dtype)) || (y && bad_dt(y_dtype)) || (z && bad_dt(z_dtype)))
    return op_fail(FR_B200_E_ARG, "dtype must be f16 or f32");
  if (op != FR_B200_EW_FILL && !x) return op_fail(FR_B200_E_ARG, "x missing");
  if ((op == FR_B200_EW_ADD || op == FR_B200_EW_MUL || op == FR_B200_EW_FMA) && !y) return op_fail(FR_B200_E_ARG, "y missing");
  if (op == FR_B200_EW_FMA && !z) return op_fail(FR_B200_E_ARG, "z missing");
  if (n == 0) return FR_B200_OK;
  elementwise_op_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(op, x, x_dtype, y, y_dtype, z,
                                                                                                        z_dtype, alpha, out, out_dtype, n);
  OP_CU(cudaGetLastError());
  return FR_B200_OK;
}

int fr_b200_matmul(const void *a, int a_dtype, int M, int K, const void *w, int w_dtype, int N, void *out, int out_dtype,
                   int device, void *stream) {
  if (!a || !w || !out || M < 1 || N < 1 || K < 64 || K % 64) return op_fail(FR_B200_E_ARG, "bad argument (K must be a positive multiple of 64)");
  if (bad_dt(a_dtype) || bad_dt(w_dtype) || bad_dt(out_dtype)) return op_fail(FR_B200_E_ARG, "dtype must be f16 or f32");
  OP_CU(cudaSetDevice(device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  OpBuf a32, w32, y32;
  const void *ap = a, *wp = w;
  int rc;
  if (a_dtype != FR_B200_T_F32) {
    OP_CU(a32.alloc((size_t)M * K * 4));
    if ((rc = fr_b200_elementwise(FR_B200_EW_COPY, a, a_dtype, nullptr, 0, nullptr, 0, 0.f, a32.p, FR_B200_T_F32, (size_t)M * K, stream))) return rc;
    ap = a32.p;
  }
  if (w_dtype != FR_B200_T_F32) {
    OP_CU(w32.alloc((size_t)K * N * 4));
    if ((rc = fr_b200_elementwise(FR_B200_EW_COPY, w, w_dtype, nullptr, 0, nullptr, 0, 0.f, w32.p, FR_B200_T_F32, (size_t)K * N, stream))) return rc;
    wp = w32.p;
  }
  OP_CU(y32.alloc((size_t)M * N * 4));
  OP_CU(cudaStreamSynchronize(st));
  // few rows: the streaming matvec (activations as fp16 hi + lo pairs); more: the tensor-core GEMM (fp16 operands)
  if (M <= 8) rc = fr_b200_matvec(reinterpret_cast<const float *>(wp), K, N, FR_B200_W_FP16, reinterpret_cast<const float *>(ap), M,
                                  reinterpret_cast<float *>(y32.p), device);
  else rc = fr_b200_gemm_f16(reinterpret_cast<const float *>(ap), reinterpret_cast<const float *>(wp), M, N, K, 0, nullptr, nullptr, 1.f,
                             reinterpret_cast<float *>(y32.p), device);
  if (rc) return op_fail(rc, fr_b200_last_error());
  if ((rc = fr_b200_elementwise(FR_B200_EW_COPY, y32.p, FR_B200_T_F32, nullptr, 0, nullptr, 0, 0.f, out, out_dtype, (size_t)M * N, stream))) return rc;
  OP_CU(cudaStreamSynchronize(st));   // the temporaries go away with this call
  return FR_B200_OK;
}

}  // extern "C"
