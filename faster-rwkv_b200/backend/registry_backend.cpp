// Registry glue: plugs the fr_b200 C ABI into the reference's kernel registry for Device::kCUDA, so that
// the reference's model.cpp / tensor.cpp / drivers run on the B200 backend unchanged.
//
// Keys registered (signatures from kernels/kernels.h):
//   "allocator"          Allocator &(*)()                                              kernels.h:286-289
//   "init_model"         void(*)(Model*, Device, const string&, const string&, const any&)   :268-272
//   "model_forward"      Tensor(*)(Model*, Device, int)                                 :274-277
//   "model_forward_seq"  Tensor(*)(Model*, Device, const vector<int>&, bool)            :279-284
//   op level             "att", "att_one_v5", "att_seq_v5", "att_one_v5_1", "att_seq_v5_2", "ffn", "ffn_seq",
//                        "layernorm", "groupnorm", "matmul", "cast_dtype", "fill_", "scalar_div_", "slice"   :15-206
// They replace def::init_model / def::ModelForward / def::ModelForwardSeq (kernels/default/*.cpp), which
// register themselves for kCUDA too; the registry keeps the last writer (kernels/registry.h:17-19), so this
// object must be linked after them, or fr_b200_backend_install() called once before the first Model.
//
// State handling: Model::ResetStates / LoadStateFile replace the state tensors wholesale (model.cpp:139,
// 145-177).  Every forward compares the tensors in model->states() with the views this backend handed out;
// foreign tensors (host or device) are imported into the backend's state first, then the views are refreshed.
// C-ABI status codes become FRException, the reference's error type (check.h:11-48).
#include <algorithm>
#include <any>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>
#include <msgpack.hpp>

#include <kernels/allocator.h>
#include <kernels/kernels.h>
#include <kernels/registry.h>
#include <tensor.h>
#define private public
#include <model.h>
#undef private

#include "../../include/fr_b200.h"

namespace rwkv {
namespace b200 {

#define FRB_CALL(expr)                                                                            \
  do {                                                                                            \
    int st_ = (expr);                                                                             \
    if (st_ < 0) throw FRException() << #expr << ": " << fr_b200_strerror(st_) << ": " << fr_b200_last_error(); \
  } while (0)

// plain device allocator for the few tensors the reference itself puts on the GPU (the initial states)
class DeviceAllocator : public Allocator {
public:
  void *DoAllocate(size_t size) override {
    void *p = nullptr;
    if (cudaMalloc(&p, size ? size : kAlignSize) != cudaSuccess) throw FRException() << "cudaMalloc failed";
    return p;
  }
  void Deallocate(void *ptr) override { cudaFree(ptr); }
};
Allocator &allocator() {
  static DeviceAllocator a;
  return a;
}

struct Extra {
  fr_b200_model *h = nullptr;
  int vocab = 0;
  std::vector<void *> views;  // device pointers last handed out through model->states()
  ~Extra() { if (h) fr_b200_destroy(h); }
};
using ExtraPtr = std::shared_ptr<Extra>;

static int version_code(const std::string &v) {
  if (v == "4") return FR_B200_V4;
  if (v == "5") return FR_B200_V5_0;
  if (v == "5.1") return FR_B200_V5_1;
  if (v == "5.2") return FR_B200_V5_2;
  RV_UNIMPLEMENTED() << "model version " << v;
}

static void upload(fr_b200_model *h, const std::string &name, const msgpack::object &obj) {
  auto m = obj.as<std::unordered_map<std::string, msgpack::object>>();
  auto data = m["data"].as<std::vector<char>>();
  auto shape = m["shape"].as<std::vector<int64_t>>();
  auto dtype = m["dtype"].as<std::string>();
  int dt;
  if (dtype == "torch.float16") dt = FR_B200_T_F16;
  else if (dtype == "torch.float32") dt = FR_B200_T_F32;
  else RV_UNIMPLEMENTED() << "tensor dtype " << dtype;
  FRB_CALL(fr_b200_set_tensor(h, name.c_str(), data.data(), dt, shape.data(), (int)shape.size()));
}

// replaces def::init_model (kernels/default/init_model.cpp:19-133): same file format, but the tensors go
// straight into the backend's packed layout instead of Model::_params
static const char *version_string(int code) {
  return code == FR_B200_V4 ? "4" : code == FR_B200_V5_0 ? "5" : code == FR_B200_V5_1 ? "5.1" : "5.2";
}

// FR_B200_CACHE=1: a packed copy of the model (<file>.b200-<fp16|int8|int4>) is written after the first load and read
// instead of the `.fr` file from then on: a few large reads in place of the msgpack parse, the upload per embedding
// row and the re-quantisation.  Returns true when the model came from the cache.
static bool load_from_cache(Model *model, const std::string &cache, int weight_format, int act_fp16) {
  std::ifstream probe(cache, std::ios::binary);
  if (!probe.good()) return false;
  probe.close();
  auto ex = std::make_shared<Extra>();
  if (fr_b200_load_packed(cache.c_str(), 1, 0, 1, &ex->h) < 0) return false;   // stale or foreign file: load the `.fr`
  fr_b200_config cfg;
  FRB_CALL(fr_b200_get_config(ex->h, &cfg));
  if (cfg.weight_format != weight_format || cfg.act_fp16 != act_fp16) return false;
  model->_n_layer = cfg.n_layer;
  model->_n_embd = cfg.n_embd;
  model->_n_att = cfg.n_embd;
  model->_n_ffn = cfg.n_ffn;
  model->_head_size = cfg.n_head;   // the reference keeps n_head in _head_size (init_model.cpp:64)
  model->_version = version_string(cfg.version);
  ex->vocab = cfg.vocab;
  model->_extra = ex;
  return true;
}

void init_model(Model *model, Device device, const std::string &path, const std::string &strategy,
                const std::any &extra) {
  int wfmt;
  if (model->_weight_dtype == DType::kFloat16) wfmt = FR_B200_W_FP16;
  else if (model->_weight_dtype == DType::kInt8) wfmt = FR_B200_W_INT8;
  else if (model->_weight_dtype == DType::kInt4) wfmt = FR_B200_W_INT4;
  else RV_UNIMPLEMENTED() << "strategy " << strategy << ": this backend implements cuda fp16 / int8 / int4";
  const char *cache_env = std::getenv("FR_B200_CACHE");
  const bool use_cache = cache_env && cache_env[0] == '1';
  const std::string cache = path + ".b200-" + (wfmt == FR_B200_W_FP16 ? "fp16" : wfmt == FR_B200_W_INT8 ? "int8" : "int4");
  if (use_cache && load_from_cache(model, cache, wfmt, model->_act_dtype == DType::kFloat16)) return;
  std::ifstream in(path, std::ios::binary | std::ios::ate);
  RV_CHECK(in.good()) << "cannot open " << path;
  const std::streamsize len = in.tellg();
  in.seekg(0);
  std::vector<char> buf(len);
  in.read(buf.data(), len);
  auto handle = msgpack::unpack(buf.data(), buf.size());
  auto map = handle.get().as<std::unordered_map<std::string, msgpack::object>>();
  auto weights = map["weights"].as<std::map<std::string, msgpack::object>>();
  auto emb = map["embd_weights"].as<std::vector<msgpack::object>>();

  model->_n_layer = map["n_layer"].as<int>();
  model->_n_embd = map["n_embd"].as<int>();
  model->_version = map.count("version") ? map["version"].as<std::string>() : std::string("4");
  if (model->_version.substr(0, 1) == "5") {
    model->_head_size = map["n_head"].as<int>();   // the reference keeps n_head in _head_size (init_model.cpp:64)
    model->_n_att = map["n_att"].as<int>();
    model->_n_ffn = map["n_ffn"].as<int>();
  } else {
    model->_n_att = model->_n_embd;
  }
  int n_ffn = model->_n_ffn;
  if (n_ffn == 0) {
    auto kw = weights["blocks.0.ffn.key.weight"].as<std::unordered_map<std::string, msgpack::object>>();
    n_ffn = (int)kw["shape"].as<std::vector<int64_t>>()[1];
  }

  fr_b200_config cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.version = version_code(model->_version);
  cfg.n_layer = model->_n_layer;
  cfg.n_embd = model->_n_embd;
  cfg.n_ffn = n_ffn;
  cfg.n_head = model->_head_size;
  cfg.vocab = (int)emb.size();
  cfg.weight_format = wfmt;
  cfg.act_fp16 = model->_act_dtype == DType::kFloat16;
  cfg.max_batch = 1;
  cfg.device = 0;
  // Model::SaveStateFile reads the state tensors with memcpy (model.cpp:110): hand out addresses the host can read
  // managed state memory, so that the unchanged Model::SaveStateFile (a plain memcpy of data_ptr(), model.cpp:110)
  // works; FR_B200_HOST_STATE=0 keeps the state in ordinary device memory (state files then need the C ABI's export)
  {
    const char *hs = std::getenv("FR_B200_HOST_STATE");
    cfg.host_visible_state = (hs && std::atoi(hs) == 0) ? 0 : 1;
  }

  auto ex = std::make_shared<Extra>();
  FRB_CALL(fr_b200_create(&cfg, &ex->h));
  ex->vocab = cfg.vocab;
  for (auto &kv : weights) upload(ex->h, kv.first, kv.second);
  for (size_t i = 0; i < emb.size(); ++i) upload(ex->h, "emb." + std::to_string(i), emb[i]);
  FRB_CALL(fr_b200_finalize(ex->h));
  if (use_cache) fr_b200_save_packed(ex->h, cache.c_str());   // best effort: an unwritable directory just means no cache
  model->_extra = ex;
}

static ExtraPtr get_extra(Model *model) {
  try {
    return std::any_cast<ExtraPtr>(model->_extra);
  } catch (const std::bad_any_cast &) {
    throw FRException() << "model was not initialised by the fr_b200 backend";
  }
}

static size_t tensor_bytes(const Tensor &t) { return (size_t)t.numel() * t.elem_size(); }

// bring model->states() and the backend's state in line (see the header comment)
static void sync_states_in(Model *model, Extra &ex) {
  auto &states = model->states();
  const int cnt = fr_b200_state_count(ex.h);
  bool mine = ex.views.size() == states.size() * (size_t)cnt;
  for (size_t l = 0; mine && l < states.size(); ++l)
    for (int j = 0; j < cnt; ++j)
      if ((int)states[l].size() != cnt || states[l][j].data_ptr() != ex.views[l * cnt + j]) { mine = false; break; }
  if (mine) return;
  RV_CHECK((int)states.size() == model->_n_layer);
  std::vector<char> flat(fr_b200_state_bytes(ex.h));
  size_t pos = 0;
  for (size_t l = 0; l < states.size(); ++l) {
    RV_CHECK((int)states[l].size() == cnt);
    for (int j = 0; j < cnt; ++j) {
      const Tensor &t = states[l][j];
      void *ptr; int dt; int64_t n;
      FRB_CALL(fr_b200_state_tensor(ex.h, 0, (int)l, j, &ptr, &dt, &n));
      RV_CHECK(t.numel() == n) << "state tensor shape mismatch";
      RV_CHECK((t.dtype() == DType::kFloat16) == (dt == FR_B200_T_F16)) << "state tensor dtype mismatch";
      const size_t bytes = tensor_bytes(t);
      RV_CHECK(pos + bytes <= flat.size());
      RV_CHECK(cudaMemcpy(flat.data() + pos, t.data_ptr(), bytes, cudaMemcpyDefault) == cudaSuccess);
      pos += bytes;
    }
  }
  RV_CHECK(pos == flat.size());
  FRB_CALL(fr_b200_state_reset(ex.h, 0));
  FRB_CALL(fr_b200_state_import(ex.h, 0, flat.data(), flat.size()));
}

// model->states() := views of the backend's current state tensors (reference shapes and dtypes)
static void publish_states(Model *model, Extra &ex) {
  auto &states = model->states();
  const int cnt = fr_b200_state_count(ex.h);
  ex.views.assign(states.size() * cnt, nullptr);
  for (size_t l = 0; l < states.size(); ++l)
    for (int j = 0; j < cnt; ++j) {
      void *ptr; int dt; int64_t n;
      FRB_CALL(fr_b200_state_tensor(ex.h, 0, (int)l, j, &ptr, &dt, &n));
      const Shape shape = states[l][j].shape();
      states[l][j] = Tensor::FromPtr(ptr, shape, dt == FR_B200_T_F16 ? DType::kFloat16 : DType::kFloat32, Device::kCUDA);
      ex.views[l * cnt + j] = ptr;
    }
}

// replaces def::ModelForward (kernels/default/model_forward.cpp:22-193).  The logits come back as a host
// fp32 tensor, which Model::Run passes through unchanged (Copy to the same device is a no-op, tensor.cpp:59-61).
Tensor model_forward(Model *model, Device device, int id) {
  auto ex = get_extra(model);
  sync_states_in(model, *ex);
  Tensor out = Tensor::Empty({(LengthType)ex->vocab}, DType::kFloat32, Device::kCPU);
  const int32_t tid = id;
  FRB_CALL(fr_b200_decode(ex->h, &tid, 1, out.data_ptr<float>(), nullptr, nullptr));
  publish_states(model, *ex);
  return out;
}

// replaces def::ModelForwardSeq (kernels/default/model_forward_seq.cpp:48-184).  RWKV-4 has no seq kernel
// upstream (it throws, :111-112); here it runs the token loop of :34-46, RWKV-5.x prompts the seq kernels.
Tensor model_forward_seq(Model *model, Device device, const std::vector<int> &ids, bool full_output) {
  RV_CHECK(!ids.empty());
  auto ex = get_extra(model);
  sync_states_in(model, *ex);
  const LengthType V = ex->vocab, T = (LengthType)ids.size();
  Tensor out = full_output ? Tensor::Empty({T, V}, DType::kFloat32, Device::kCPU)
                           : Tensor::Empty({V}, DType::kFloat32, Device::kCPU);
  if (!full_output) {
    // the whole prompt at once: RWKV-5.x with fp16 weights runs the seq kernels, everything else the token loop
    std::vector<int32_t> tids(ids.begin(), ids.end());
    FRB_CALL(fr_b200_run_seq(ex->h, 0, tids.data(), (int)T, out.data_ptr<float>(), nullptr));
  } else {
    for (LengthType t = 0; t < T; ++t) {
      const int32_t tid = ids[t];
      FRB_CALL(fr_b200_decode(ex->h, &tid, 1, out.data_ptr<float>() + t * V, nullptr, nullptr));
    }
  }
  publish_states(model, *ex);
  return out;
}

// ---- op-level keys (kernels/kernels.h:15-257) ------------------------------------------------------------------
// The reference's own layer loop (def::ModelForward / def::ModelForwardSeq, kernels/default/model_forward*.cpp) calls
// these per op; they are thin calls into the stand-alone operator entry points of the C ABI.  With the model-level
// keys above installed the drivers never reach them; FR_B200_OP_LEVEL=1 leaves the model-level keys to the
// reference's default implementations so that its loop runs over these operators (tests/test_gpu_dropin.py).
namespace ops {

#define FRB_OP(expr)                                                                                \
  do {                                                                                              \
    int st_ = (expr);                                                                               \
    if (st_ < 0) throw FRException() << #expr << ": " << fr_b200_strerror(st_) << ": " << fr_b200_op_last_error(); \
  } while (0)

static int dt(const Tensor &t) {
  if (t.dtype() == DType::kFloat16) return FR_B200_T_F16;
  if (t.dtype() == DType::kFloat32) return FR_B200_T_F32;
  RV_UNIMPLEMENTED() << "tensor dtype " << dtype_to_string(t.dtype());
}
static Tensor empty(const Shape &shape, DType dtype) { return Tensor::Empty(shape, dtype, Device::kCUDA); }
static void ew(int op, const Tensor *x, const Tensor *y, const Tensor *z, float alpha, Tensor &out) {
  FRB_OP(fr_b200_elementwise(op, x ? x->data_ptr() : nullptr, x ? dt(*x) : 0, y ? y->data_ptr() : nullptr, y ? dt(*y) : 0,
                             z ? z->data_ptr() : nullptr, z ? dt(*z) : 0, alpha, out.data_ptr(), dt(out), (size_t)out.numel(), nullptr));
}
// a [K] or [M, K] times w [K, N]
static Tensor mm(const Tensor &a, const Tensor &w, DType out_dtype) {
  RV_CHECK(w.shape().size() == 2);
  const LengthType K = w.size(0), N = w.size(1);
  RV_CHECK(a.shape().size() >= 1 && a.shape().back() == K) << "matmul shapes";
  const LengthType M = a.numel() / K;
  Shape os = a.shape();
  os.back() = N;
  Tensor out = empty(os, out_dtype);
  FRB_OP(fr_b200_matmul(a.data_ptr(), dt(a), (int)M, (int)K, w.data_ptr(), dt(w), (int)N, out.data_ptr(), dt(out), 0, nullptr));
  return out;
}
// LayerNorm + token-shift mix of `rows` rows against the shift rows `sx` (same shape): xx and fp32 mixed vectors
static Tensor ln_mix(const Tensor &x, const Tensor &sx, const Tensor &ln_w, const Tensor &ln_b, const std::vector<const Tensor *> &mix,
                     std::vector<Tensor> &out) {
  const LengthType C = ln_w.numel(), rows = x.numel() / C;
  Tensor xx = empty(x.shape(), x.dtype());
  const void *mp[4] = {nullptr, nullptr, nullptr, nullptr};
  void *op[4] = {nullptr, nullptr, nullptr, nullptr};
  out.clear();
  for (size_t v = 0; v < mix.size(); ++v) {
    out.push_back(empty(x.shape(), DType::kFloat32));
    mp[v] = mix[v]->data_ptr();
    op[v] = out.back().data_ptr();
  }
  FRB_OP(fr_b200_ln_mix(x.data_ptr(), mix.empty() ? nullptr : sx.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(), mp, (int)mix.size(),
                        (int)rows, (int)C, dt(x), dt(ln_w), FR_B200_T_F32, xx.data_ptr(), op, nullptr));
  return xx;
}
// seq mode: row t mixes against xx[t - 1], row 0 against the stored shift state (att_seq.cu:377-381, ffn_seq.cu:70-76)
// returns the new shift state: xx of the last row
static Tensor ln_mix_rows(const Tensor &x, const Tensor &sx, const Tensor &ln_w, const Tensor &ln_b,
                          const std::vector<const Tensor *> &mix, std::vector<Tensor> &out) {
  const LengthType C = ln_w.numel(), T = x.numel() / C;
  if (T == 1) return ln_mix(x, sx, ln_w, ln_b, mix, out);
  std::vector<Tensor> none;
  Tensor xx = ln_mix(x, sx, ln_w, ln_b, {}, none);
  Tensor shifted = empty(x.shape(), x.dtype());
  const size_t rb = (size_t)C * x.elem_size();
  RV_CHECK(cudaMemcpy(shifted.data_ptr(), sx.data_ptr(), rb, cudaMemcpyDeviceToDevice) == cudaSuccess);
  if (T > 1) RV_CHECK(cudaMemcpy(static_cast<char *>(shifted.data_ptr()) + rb, xx.data_ptr(), rb * (T - 1), cudaMemcpyDeviceToDevice) == cudaSuccess);
  Tensor last_xx = empty({C}, x.dtype());
  RV_CHECK(cudaMemcpy(last_xx.data_ptr(), static_cast<const char *>(xx.data_ptr()) + rb * (T - 1), rb, cudaMemcpyDeviceToDevice) == cudaSuccess);
  ln_mix(x, shifted, ln_w, ln_b, mix, out);
  return last_xx;
}

// "att": kernels/kernels.h:15-24, kernels/cuda/att.cu:337-359 (RWKV-4, one token)
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor>
att(const Tensor &x, const Tensor &sx, const Tensor &aa, const Tensor &bb, const Tensor &pp, const Tensor &ln_w, const Tensor &ln_b,
    const Tensor &k_mix, const Tensor &v_mix, const Tensor &r_mix, const Tensor &t_decay, const Tensor &t_first, const Tensor &kw,
    const Tensor &vw, const Tensor &rw, const Tensor &ow) {
  std::vector<Tensor> mixed;
  Tensor xx = ln_mix(x, sx, ln_w, ln_b, {&k_mix, &v_mix, &r_mix}, mixed);
  Tensor k = mm(mixed[0], kw, DType::kFloat32), v = mm(mixed[1], vw, DType::kFloat32), r = mm(mixed[2], rw, DType::kFloat32);
  const LengthType C = x.numel();
  Tensor rwkv = empty({C}, DType::kFloat32), aa2 = empty(aa.shape(), DType::kFloat32), bb2 = empty(bb.shape(), DType::kFloat32),
         pp2 = empty(pp.shape(), DType::kFloat32);
  FRB_OP(fr_b200_wkv4_step(k.data_ptr<float>(), v.data_ptr<float>(), r.data_ptr<float>(), t_decay.data_ptr<float>(),
                           t_first.data_ptr<float>(), aa.data_ptr<float>(), bb.data_ptr<float>(), pp.data_ptr<float>(), (int)C,
                           FR_B200_T_F32, rwkv.data_ptr(), aa2.data_ptr<float>(), bb2.data_ptr<float>(), pp2.data_ptr<float>(), nullptr));
  Tensor o = mm(rwkv, ow, DType::kFloat32);
  Tensor xo = empty(x.shape(), x.dtype());
  ew(FR_B200_EW_ADD, &x, &o, nullptr, 0.f, xo);
  return {xo, xx, aa2, bb2, pp2};
}

// shared by the RWKV-5 keys: rows = 1 (one token) or T (seq mode)
static std::tuple<Tensor, Tensor, Tensor> att_v5(const Tensor &x, const Tensor &sx, const Tensor &s, const Tensor &ln_w, const Tensor &ln_b,
                                                 const Tensor &lx_w, const Tensor &lx_b, const std::vector<const Tensor *> &mix,
                                                 const Tensor &t_decay, const Tensor &t_first, const Tensor &kw, const Tensor &vw,
                                                 const Tensor &rw, const Tensor *gw, const Tensor &ow) {
  const LengthType C = ln_w.numel(), T = x.numel() / C, H = s.size(0);
  RV_CHECK(C == H * 64) << "head size must be 64";
  std::vector<Tensor> mixed;
  Tensor xx_state = ln_mix_rows(x, sx, ln_w, ln_b, mix, mixed);
  Tensor k = mm(mixed[0], kw, DType::kFloat32), v = mm(mixed[1], vw, DType::kFloat32), r = mm(mixed[2], rw, DType::kFloat32);
  const int per_head = t_decay.numel() == H;
  Tensor y = empty(k.shape(), DType::kFloat32), s2 = empty(s.shape(), DType::kFloat32);
  if (T == 1) {
    FRB_OP(fr_b200_wkv5_step(r.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(), t_decay.data_ptr<float>(),
                             t_first.data_ptr<float>(), per_head, s.data_ptr<float>(), (int)H, s2.data_ptr<float>(), y.data_ptr<float>(),
                             nullptr));
  } else {
    RV_CHECK(cudaMemcpy(s2.data_ptr(), s.data_ptr(), (size_t)s.numel() * 4, cudaMemcpyDeviceToDevice) == cudaSuccess);
    const int n_chunks = (int)std::max<LengthType>(1, T / 32);
    FRB_OP(fr_b200_wkv5_chunk_scan(r.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(), t_decay.data_ptr<float>(),
                                   t_first.data_ptr<float>(), per_head, s2.data_ptr<float>(), (int)H, (int)T, n_chunks,
                                   y.data_ptr<float>(), nullptr));
  }
  Tensor yn = empty(y.shape(), DType::kFloat32);
  FRB_OP(fr_b200_groupnorm(y.data_ptr(), lx_w.data_ptr(), lx_b.data_ptr(), (int)T, (int)C, (int)H, FR_B200_T_F32, dt(lx_w), yn.data_ptr(),
                           nullptr));
  if (gw) {
    Tensor g = mm(mixed[3], *gw, DType::kFloat32);
    ew(FR_B200_EW_SILU, &g, nullptr, nullptr, 0.f, g);
    ew(FR_B200_EW_MUL, &yn, &g, nullptr, 0.f, yn);
  }
  Tensor o = mm(yn, ow, DType::kFloat32);
  Tensor xo = empty(x.shape(), x.dtype());
  ew(FR_B200_EW_ADD, &x, &o, nullptr, 0.f, xo);
  return {xo, xx_state, s2};
}

// "att_one_v5" / "att_seq_v5": kernels/kernels.h:26-50, kernels/cuda/att.cu:361-391, att_seq.cu:425-462
std::tuple<Tensor, Tensor, Tensor> att_v5_0(const Tensor &x, const Tensor &sx, const Tensor &s, const Tensor &ln_w, const Tensor &ln_b,
                                            const Tensor &lx_w, const Tensor &lx_b, const Tensor &k_mix, const Tensor &v_mix,
                                            const Tensor &r_mix, const Tensor &t_decay, const Tensor &t_first, const Tensor &kw,
                                            const Tensor &vw, const Tensor &rw, const Tensor &ow) {
  return att_v5(x, sx, s, ln_w, ln_b, lx_w, lx_b, {&k_mix, &v_mix, &r_mix}, t_decay, t_first, kw, vw, rw, nullptr, ow);
}
// "att_one_v5_1": kernels/kernels.h:52-63, kernels/cuda/att.cu:393-425
std::tuple<Tensor, Tensor, Tensor> att_v5_1(const Tensor &x, const Tensor &sx, const Tensor &s, const Tensor &ln_w, const Tensor &ln_b,
                                            const Tensor &lx_w, const Tensor &lx_b, const Tensor &k_mix, const Tensor &v_mix,
                                            const Tensor &r_mix, const Tensor &g_mix, const Tensor &t_decay, const Tensor &t_first,
                                            const Tensor &kw, const Tensor &vw, const Tensor &rw, const Tensor &gw, const Tensor &ow) {
  return att_v5(x, sx, s, ln_w, ln_b, lx_w, lx_b, {&k_mix, &v_mix, &r_mix, &g_mix}, t_decay, t_first, kw, vw, rw, &gw, ow);
}
// "att_seq_v5_2": kernels/kernels.h:65-76, kernels/cuda/att_seq.cu:464-493
std::tuple<Tensor, Tensor, Tensor> att_seq_v5_2(const Tensor &x, const Tensor &sx, const Tensor &s, const Tensor &ln_w, const Tensor &ln_b,
                                                const Tensor &lx_w, const Tensor &lx_b, const Tensor &k_mix, const Tensor &v_mix,
                                                const Tensor &r_mix, const Tensor &g_mix, const Tensor &t_decay, const Tensor &t_first,
                                                const Tensor &kw, const Tensor &vw, const Tensor &rw, const Tensor &gw, const Tensor &ow,
                                                int n_att) {
  (void)n_att;
  return att_v5(x, sx, s, ln_w, ln_b, lx_w, lx_b, {&k_mix, &v_mix, &r_mix, &g_mix}, t_decay, t_first, kw, vw, rw, &gw, ow);
}

// "ffn" / "ffn_seq": kernels/kernels.h:80-96, kernels/cuda/ffn.cu:89-110, ffn_seq.cu:89-109
std::tuple<Tensor, Tensor> ffn(const Tensor &x, const Tensor &sx, const Tensor &ln_w, const Tensor &ln_b, const Tensor &k_mix,
                               const Tensor &r_mix, const Tensor &kw, const Tensor &vw, const Tensor &rw) {
  const LengthType C = ln_w.numel(), T = x.numel() / C;
  std::vector<Tensor> mixed;
  Tensor xx_state = ln_mix_rows(x, sx, ln_w, ln_b, {&k_mix, &r_mix}, mixed);
  Tensor k = mm(mixed[0], kw, DType::kFloat32), r = mm(mixed[1], rw, DType::kFloat32);
  ew(FR_B200_EW_RELU2, &k, nullptr, nullptr, 0.f, k);
  ew(FR_B200_EW_SIGMOID, &r, nullptr, nullptr, 0.f, r);
  Tensor vk = mm(k, vw, DType::kFloat32);
  Tensor xo = empty(x.shape(), x.dtype());
  ew(FR_B200_EW_FMA, &r, &vk, &x, 0.f, xo);
  return {xo, xx_state};
}

// "layernorm", "groupnorm", "matmul", "cast_dtype", "fill_", "scalar_div_": kernels/kernels.h:98-128
Tensor layernorm(const Tensor &x, const Tensor &weight, const Tensor &bias) {
  std::vector<Tensor> none;
  return ln_mix(x, x, weight, bias, {}, none);
}
Tensor groupnorm(const Tensor &x, int num_groups, const Tensor &weight, const Tensor &bias) {
  const LengthType C = weight.numel();
  Tensor out = empty(x.shape(), x.dtype());
  FRB_OP(fr_b200_groupnorm(x.data_ptr(), weight.data_ptr(), bias.data_ptr(), (int)(x.numel() / C), (int)C, num_groups, dt(x), dt(weight),
                           out.data_ptr(), nullptr));
  return out;
}
Tensor matmul(const Tensor &a, const Tensor &b) {
  RV_CHECK(b.shape().size() == 2 && a.shape().size() <= 2) << "the B200 operator path multiplies [K] or [M, K] by [K, N]";
  return mm(a, b, a.dtype());
}
Tensor cast_dtype(const Tensor &x, DType dtype) {
  Tensor out = empty(x.shape(), dtype);
  ew(FR_B200_EW_COPY, &x, nullptr, nullptr, 0.f, out);
  return out;
}
Tensor &fill_(Tensor &x, float val) {
  ew(FR_B200_EW_FILL, nullptr, nullptr, nullptr, val, x);
  return x;
}
Tensor scalar_div_(Tensor &x, float val) {
  ew(FR_B200_EW_SCALE, &x, nullptr, nullptr, 1.f / val, x);
  return x;
}

// "slice": kernels/kernels.h:203-206, kernels/cuda/slice.cu:41-117.  Ranges of whole rows (a unit-stride range on the first
// dimension, everything else taken whole) are one device copy; that is what the reference's layer loops ask for
// (the last prompt row, kernels/default/model_forward_seq.cpp:171).
Tensor slice(const Tensor &x, const std::vector<Range> &ranges) {
  RV_CHECK(x.shape().size() == ranges.size() && !ranges.empty());
  for (size_t d = 1; d < ranges.size(); ++d) {
    const Range &r = ranges[d];
    RV_CHECK((r.start == 0 && r.interval == 0 && r.end == 0) || (r.start == 0 && r.interval == 1 && r.end == x.size(d)))
        << "the B200 operator path slices whole rows only";
  }
  LengthType start = ranges[0].start, end = ranges[0].end, n0 = x.size(0);
  int interval = ranges[0].interval;
  if (start == 0 && interval == 0 && end == 0) { end = n0; interval = 1; }
  if (start < 0) start += n0;
  if (end < 0) end += n0;
  RV_CHECK(interval == 1 && start <= end && end <= n0) << "the B200 operator path slices unit-stride row ranges only";
  Shape os = x.shape();
  os[0] = end - start;
  Tensor out = empty(os, x.dtype());
  const size_t row_bytes = (size_t)(x.numel() / n0) * x.elem_size();
  if (end > start)
    RV_CHECK(cudaMemcpy(out.data_ptr(), static_cast<const char *>(x.data_ptr()) + (size_t)start * row_bytes,
                        (size_t)(end - start) * row_bytes, cudaMemcpyDeviceToDevice) == cudaSuccess);
  return out;
}

}  // namespace ops

void install() {
  auto &r = KernelRegistry::Instance();
  r.Register("allocator", Device::kCUDA, allocator, 1);
  const char *op_level = std::getenv("FR_B200_OP_LEVEL");
  if (!(op_level && op_level[0] == '1')) {
    r.Register("init_model", Device::kCUDA, init_model, 1);
    r.Register("model_forward", Device::kCUDA, model_forward, 1);
    r.Register("model_forward_seq", Device::kCUDA, model_forward_seq, 1);
  }
  r.Register("att", Device::kCUDA, ops::att, 1);
  r.Register("att_one_v5", Device::kCUDA, ops::att_v5_0, 1);
  r.Register("att_seq_v5", Device::kCUDA, ops::att_v5_0, 1);
  r.Register("att_one_v5_1", Device::kCUDA, ops::att_v5_1, 1);
  r.Register("att_seq_v5_2", Device::kCUDA, ops::att_seq_v5_2, 1);
  r.Register("ffn", Device::kCUDA, ops::ffn, 1);
  r.Register("ffn_seq", Device::kCUDA, ops::ffn, 1);
  r.Register("layernorm", Device::kCUDA, ops::layernorm, 1);
  r.Register("groupnorm", Device::kCUDA, ops::groupnorm, 1);
  r.Register("matmul", Device::kCUDA, ops::matmul, 1);
  r.Register("cast_dtype", Device::kCUDA, ops::cast_dtype, 1);
  r.Register("fill_", Device::kCUDA, ops::fill_, 1);
  r.Register("scalar_div_", Device::kCUDA, ops::scalar_div_, 1);
  r.Register("slice", Device::kCUDA, ops::slice, 1);
}

namespace {
struct AutoInstall {
  AutoInstall() { install(); }
} auto_install;
}  // namespace

}  // namespace b200
}  // namespace rwkv

extern "C" void fr_b200_backend_install(void) { rwkv::b200::install(); }
