// Registry glue: plugs the fr_b200 C ABI into the reference's kernel registry for Device::kCUDA, so that
// the reference's model.cpp / tensor.cpp / drivers run on the B200 backend unchanged.
//
// Keys registered (signatures from kernels/kernels.h):
//   "allocator"          Allocator &(*)()                                              kernels.h:286-289
//   "init_model"         void(*)(Model*, Device, const string&, const string&, const any&)   :268-272
//   "model_forward"      Tensor(*)(Model*, Device, int)                                 :274-277
//   "model_forward_seq"  Tensor(*)(Model*, Device, const vector<int>&, bool)            :279-284
// They replace def::init_model / def::ModelForward / def::ModelForwardSeq (kernels/default/*.cpp), which
// register themselves for kCUDA too; the registry keeps the last writer (kernels/registry.h:17-19), so this
// object must be linked after them, or fr_b200_backend_install() called once before the first Model.
//
// State handling: Model::ResetStates / LoadStateFile replace the state tensors wholesale (model.cpp:139,
// 145-177).  Every forward compares the tensors in model->states() with the views this backend handed out;
// foreign tensors (host or device) are imported into the backend's state first, then the views are refreshed.
// C-ABI status codes become FRException, the reference's error type (check.h:11-48).
#include <any>
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
void init_model(Model *model, Device device, const std::string &path, const std::string &strategy,
                const std::any &extra) {
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
  if (model->_weight_dtype == DType::kFloat16) cfg.weight_format = FR_B200_W_FP16;
  else if (model->_weight_dtype == DType::kInt8) cfg.weight_format = FR_B200_W_INT8;
  else if (model->_weight_dtype == DType::kInt4) cfg.weight_format = FR_B200_W_INT4;
  else RV_UNIMPLEMENTED() << "strategy " << strategy << ": this backend implements cuda fp16 / int8 / int4";
  cfg.act_fp16 = model->_act_dtype == DType::kFloat16;
  cfg.max_batch = 1;
  cfg.device = 0;

  auto ex = std::make_shared<Extra>();
  FRB_CALL(fr_b200_create(&cfg, &ex->h));
  ex->vocab = cfg.vocab;
  for (auto &kv : weights) upload(ex->h, kv.first, kv.second);
  for (size_t i = 0; i < emb.size(); ++i) upload(ex->h, "emb." + std::to_string(i), emb[i]);
  FRB_CALL(fr_b200_finalize(ex->h));
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

void install() {
  auto &r = KernelRegistry::Instance();
  r.Register("allocator", Device::kCUDA, allocator, 1);
  r.Register("init_model", Device::kCUDA, init_model, 1);
  r.Register("model_forward", Device::kCUDA, model_forward, 1);
  r.Register("model_forward_seq", Device::kCUDA, model_forward_seq, 1);
}

namespace {
struct AutoInstall {
  AutoInstall() { install(); }
} auto_install;
}  // namespace

}  // namespace b200
}  // namespace rwkv

extern "C" void fr_b200_backend_install(void) { rwkv::b200::install(); }
