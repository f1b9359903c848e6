// fp32 CPU primitives the reference does not ship.  TEST INFRASTRUCTURE ONLY.
//
// The reference registers att / ffn / layernorm / matmul / element-wise ops for CUDA and the exporters
// only (kernels/cuda/att.cu:427-429, kernels/default/att.cpp:115-117), so `Model(path, "cpu fp32")`
// throws "kernel att not found".  This translation unit registers, for Device::kCPU, the reference's own
// op compositions (def::att, def::att_one_v5, def::att_one_v5_1, def::ffn from kernels/default/att.cpp and
// ffn.cpp, linked from the reference tree unchanged) plus plain fp32 loops for the primitives those
// compositions call.  With it the reference's model.cpp + kernels/default/model_forward.cpp run on the CPU
// and produce the golden vectors that pin oracle/rwkv_oracle.c.
#include <cmath>
#include <cstring>
#include <functional>
#include <tuple>

#include <kernels/kernels.h>
#include <kernels/registry.h>
#include <tensor.h>

namespace rwkv {
namespace def {
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor>
att(const Tensor &x, const Tensor &sx, const Tensor &aa, const Tensor &bb, const Tensor &pp, const Tensor &ln_w,
    const Tensor &ln_b, const Tensor &k_mix, const Tensor &v_mix, const Tensor &r_mix, const Tensor &t_decay,
    const Tensor &t_first, const Tensor &kw, const Tensor &vw, const Tensor &rw, const Tensor &ow);
std::tuple<Tensor, Tensor, Tensor>
att_one_v5(const Tensor &x, const Tensor &sx, const Tensor &s, const Tensor &ln_w, const Tensor &ln_b,
           const Tensor &lx_w, const Tensor &lx_b, const Tensor &k_mix, const Tensor &v_mix, const Tensor &r_mix,
           const Tensor &t_decay, const Tensor &t_first, const Tensor &kw, const Tensor &vw, const Tensor &rw,
           const Tensor &ow);
std::tuple<Tensor, Tensor, Tensor>
att_one_v5_1(const Tensor &x, const Tensor &sx, const Tensor &s, const Tensor &ln_w, const Tensor &ln_b,
             const Tensor &lx_w, const Tensor &lx_b, const Tensor &k_mix, const Tensor &v_mix, const Tensor &r_mix,
             const Tensor &g_mix, const Tensor &t_decay, const Tensor &t_first, const Tensor &kw, const Tensor &vw,
             const Tensor &rw, const Tensor &gw, const Tensor &ow);
std::tuple<Tensor, Tensor> ffn(const Tensor &x, const Tensor &sx, const Tensor &ln_w, const Tensor &ln_b,
                               const Tensor &k_mix, const Tensor &r_mix, const Tensor &kw, const Tensor &vw,
                               const Tensor &rw);
}  // namespace def

namespace cpuref {

static void need_f32(const Tensor &t) { RV_CHECK(t.dtype() == DType::kFloat32) << "cpu fp32 reference needs fp32 tensors"; }

// numpy-style broadcasting of two shapes aligned at the trailing dimension
static Shape broadcast_shape(const Shape &a, const Shape &b) {
  const size_t n = std::max(a.size(), b.size());
  Shape out(n);
  for (size_t i = 0; i < n; ++i) {
    const LengthType da = i < n - a.size() ? 1 : a[i - (n - a.size())];
    const LengthType db = i < n - b.size() ? 1 : b[i - (n - b.size())];
    RV_CHECK(da == db || da == 1 || db == 1);
    out[i] = std::max(da, db);
  }
  return out;
}
static LengthType bindex(const Shape &out, const Shape &in, LengthType flat) {
  // flat index into `out` -> flat index into the (broadcast) `in`
  const size_t n = out.size(), off = n - in.size();
  LengthType idx = 0, stride = 1;
  for (size_t d = n; d-- > 0;) {
    const LengthType c = flat % out[d];
    flat /= out[d];
    if (d >= off) {
      const LengthType sz = in[d - off];
      if (sz != 1) idx += c * stride;
      stride *= sz;
    }
  }
  return idx;
}
template <typename F> static Tensor binary(const Tensor &a, const Tensor &b, F f) {
  need_f32(a); need_f32(b);
  const Shape os = broadcast_shape(a.shape(), b.shape());
  Tensor out = Tensor::Empty(os, DType::kFloat32, Device::kCPU);
  const float *pa = a.data_ptr<float>(), *pb = b.data_ptr<float>();
  float *po = out.data_ptr<float>();
  const LengthType n = out.numel();
  if (a.shape() == b.shape()) {
    for (LengthType i = 0; i < n; ++i) po[i] = f(pa[i], pb[i]);
  } else {
    for (LengthType i = 0; i < n; ++i) po[i] = f(pa[bindex(os, a.shape(), i)], pb[bindex(os, b.shape(), i)]);
  }
  return out;
}
template <typename F> static Tensor unary(const Tensor &a, F f) {
  need_f32(a);
  Tensor out = Tensor::Empty(a.shape(), DType::kFloat32, Device::kCPU);
  const float *pa = a.data_ptr<float>();
  float *po = out.data_ptr<float>();
  for (LengthType i = 0, n = a.numel(); i < n; ++i) po[i] = f(pa[i]);
  return out;
}

Tensor add(const Tensor &a, const Tensor &b) { return binary(a, b, [](float x, float y) { return x + y; }); }
Tensor sub(const Tensor &a, const Tensor &b) { return binary(a, b, [](float x, float y) { return x - y; }); }
Tensor mul(const Tensor &a, const Tensor &b) { return binary(a, b, [](float x, float y) { return x * y; }); }
Tensor div(const Tensor &a, const Tensor &b) { return binary(a, b, [](float x, float y) { return x / y; }); }
Tensor maximum(const Tensor &a, const Tensor &b) { return binary(a, b, [](float x, float y) { return x > y ? x : y; }); }
Tensor rsub_scalar(float s, const Tensor &a) { return unary(a, [s](float x) { return s - x; }); }
Tensor exp(const Tensor &a) { return unary(a, [](float x) { return std::exp(x); }); }
Tensor relu(const Tensor &a) { return unary(a, [](float x) { return x > 0.f ? x : 0.f; }); }
Tensor sigmoid(const Tensor &a) { return unary(a, [](float x) { return 1.f / (1.f + std::exp(-x)); }); }
Tensor silu(const Tensor &a) { return unary(a, [](float x) { return x / (1.f + std::exp(-x)); }); }
Tensor scalar_div_(Tensor &x, float v) {
  need_f32(x);
  float *p = x.data_ptr<float>();
  for (LengthType i = 0, n = x.numel(); i < n; ++i) p[i] /= v;
  return x;
}

// LayerNorm over the last dimension, eps 1e-5 (kernels/cuda/layer_norm.cu:101-130)
static void ln_rows(const float *x, const float *g, const float *b, LengthType rows, LengthType n, LengthType goff_stride,
                    float *y) {
  for (LengthType r = 0; r < rows; ++r) {
    const float *xr = x + r * n;
    double mean = 0, var = 0;
    for (LengthType i = 0; i < n; ++i) mean += xr[i];
    mean /= n;
    for (LengthType i = 0; i < n; ++i) { double d = xr[i] - mean; var += d * d; }
    var /= n;
    const float inv = static_cast<float>(1.0 / std::sqrt(var + 1e-5)), m = static_cast<float>(mean);
    const float *gr = g + r * goff_stride, *br = b + r * goff_stride;
    for (LengthType i = 0; i < n; ++i) y[r * n + i] = (xr[i] - m) * inv * gr[i] + br[i];
  }
}
Tensor layernorm(const Tensor &x, const Tensor &w, const Tensor &b) {
  need_f32(x); need_f32(w); need_f32(b);
  const LengthType n = x.shape().back(), rows = x.numel() / n;
  Tensor out = Tensor::Empty(x.shape(), DType::kFloat32, Device::kCPU);
  ln_rows(x.data_ptr<float>(), w.data_ptr<float>(), b.data_ptr<float>(), rows, n, 0, out.data_ptr<float>());
  return out;
}
// GroupNorm of a [m, k] input into num_groups groups per row, per-channel affine (kernels/cuda/group_norm.cu:322-357)
Tensor groupnorm(const Tensor &x, int num_groups, const Tensor &w, const Tensor &b) {
  need_f32(x); need_f32(w); need_f32(b);
  const LengthType k = x.shape().back(), m = x.numel() / k, gs = k / num_groups;
  Tensor out = Tensor::Empty(x.shape(), DType::kFloat32, Device::kCPU);
  for (LengthType r = 0; r < m; ++r)
    ln_rows(x.data_ptr<float>() + r * k, w.data_ptr<float>(), b.data_ptr<float>(), num_groups, gs, gs,
            out.data_ptr<float>() + r * k);
  return out;
}
// C = A . B for 1-D x 2-D, 2-D x 2-D and batched 3-D x 3-D (kernels/cuda/matmul.cpp:124-146)
Tensor matmul(const Tensor &a, const Tensor &b) {
  need_f32(a); need_f32(b);
  const Shape &as = a.shape(), &bs = b.shape();
  LengthType batch = 1, M, K, N;
  Shape os;
  if (as.size() == 1 && bs.size() == 2) { M = 1; K = as[0]; N = bs[1]; os = {N}; }
  else if (as.size() == 2 && bs.size() == 2) { M = as[0]; K = as[1]; N = bs[1]; os = {M, N}; }
  else { RV_CHECK(as.size() == 3 && bs.size() == 3 && as[0] == bs[0]); batch = as[0]; M = as[1]; K = as[2]; N = bs[2]; os = {batch, M, N}; }
  RV_CHECK(bs[bs.size() - 2] == K);
  Tensor out = Tensor::Empty(os, DType::kFloat32, Device::kCPU);
  const float *pa = a.data_ptr<float>(), *pb = b.data_ptr<float>();
  float *po = out.data_ptr<float>();
  for (LengthType t = 0; t < batch; ++t)
    for (LengthType m = 0; m < M; ++m) {
      float *c = po + (t * M + m) * N;
      for (LengthType n = 0; n < N; ++n) c[n] = 0.f;
      for (LengthType k = 0; k < K; ++k) {
        const float av = pa[(t * M + m) * K + k];
        const float *br = pb + (t * K + k) * N;
        for (LengthType n = 0; n < N; ++n) c[n] += av * br[n];
      }
    }
  return out;
}

KernelRegister r_add("add", Device::kCPU, add);
KernelRegister r_sub("sub", Device::kCPU, sub);
KernelRegister r_mul("mul", Device::kCPU, mul);
KernelRegister r_div("div", Device::kCPU, div);
KernelRegister r_max("maximum", Device::kCPU, maximum);
KernelRegister r_rsub("rsub_scalar", Device::kCPU, rsub_scalar);
KernelRegister r_exp("exp", Device::kCPU, exp);
KernelRegister r_relu("relu", Device::kCPU, relu);
KernelRegister r_sig("sigmoid", Device::kCPU, sigmoid);
KernelRegister r_silu("silu", Device::kCPU, silu);
KernelRegister r_sdiv("scalar_div_", Device::kCPU, scalar_div_);
KernelRegister r_ln("layernorm", Device::kCPU, layernorm);
KernelRegister r_gn("groupnorm", Device::kCPU, groupnorm);
KernelRegister r_mm("matmul", Device::kCPU, matmul);
// the reference's own compositions, now also reachable from the CPU device
KernelRegister r_att("att", Device::kCPU, def::att);
KernelRegister r_att5("att_one_v5", Device::kCPU, def::att_one_v5);
KernelRegister r_att51("att_one_v5_1", Device::kCPU, def::att_one_v5_1);
KernelRegister r_ffn("ffn", Device::kCPU, def::ffn);

}  // namespace cpuref
}  // namespace rwkv
