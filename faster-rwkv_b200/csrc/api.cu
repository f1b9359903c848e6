// C-ABI implementation (include/fr_b200.h): model memory, tensor upload + repacking, the phase
// table, decode launches, recurrent-state access.  No PyTorch types, no exceptions across the ABI.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "../../include/fr_b200.h"
#include "internal.h"

using namespace frb;

namespace {

thread_local std::string g_err;

int fail(int code, const std::string &msg) {
  g_err = msg;
  return code;
}
#define CU(call)                                                                                   \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess)                                                                         \
      return fail(FR_B200_E_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_) + " (" __FILE__ ":" + \
                                      std::to_string(__LINE__) + ")");                             \
  } while (0)

struct MatrixSlot {       // where a projection matrix lives inside the packed weight blob
  size_t tile_off = 0;    // byte offset of its first row block
  size_t item_stride = 0; // bytes between consecutive row blocks
  size_t rscale_off = 0;  // element offset into the row-scale array (int8)
  size_t rscale_stride = 0;
  int K = 0, N = 0;
  bool set = false;
  bool has_plain = false; // seq mode keeps the matrix a second time as W^T [N, K] fp16 row-major
  size_t plain_off = 0;   // offset of that copy in halfs
  size_t pscale_off = 0;  // int8: offset of the [N] output-row scales that go with the copy (the copy holds the codes)
  size_t q_off = 0;       // int8 / int4: byte offset of the row-major packed copy ([N, K] codes or [N, K/2] nibbles)
  size_t qs_off = 0;      // int4: offset (halfs) of its [N, K/32] group scales
};

struct VecSlot {
  size_t off = 0;  // float offset into the vector blob
  int n = 0;
  bool set = false;
};

}  // namespace

struct fr_b200_model {
  fr_b200_config cfg;
  int C, F, V, Vpad, L, H, fmt;
  bool v5 = false, gate = false;
  int device = 0;
  // device memory
  uint8_t *d_weights = nullptr;  size_t weights_bytes = 0;
  __half *d_rscale = nullptr;    size_t rscale_n = 0;
  float *d_vecs = nullptr;       size_t vecs_n = 0;
  __half *d_vecs16 = nullptr;    // fp16 image of d_vecs, kept when LayerNorm / mix vectors are all exact in fp16
  uint8_t *d_emb = nullptr;      int emb_dtype = -1;   // rows kept in the dtype they arrive in
  uint8_t *d_state = nullptr;    size_t state_stride = 0, layer_stride = 0;
  exch_t *d_x = nullptr, *d_xa = nullptr, *d_rwkv = nullptr, *d_kk = nullptr, *d_rr = nullptr;   // tagged exchange vectors
  exch_t *d_v5buf = nullptr;     // k5, v5, r5, g5, o5
  int exch_batch = 0;            // streams the last launch wrote into the exchange vectors (0: clear them first)
  unsigned seq = 0;              // phases launched so far (tags continue across launches)
  std::vector<unsigned> par;     // per stream slot: which copy of the token-shift states it reads next
  float *d_out = nullptr;        // [B][Vpad] logits, then [B] argmax ints, then status int
  LayerDev *d_layers = nullptr;
  PhaseDev *d_phases = nullptr;
  uint8_t *h_out = nullptr;      // pinned mirror of d_out
  unsigned long long *d_hist = nullptr; size_t hist_n = 0;   // packed arg-max words of decode_greedy, [tokens][batch]
  unsigned long long *d_amax = nullptr;   // packed arg-max words of a single decode, [max_batch]
  // GEMM path: row copies of the projection matrices, activation buffers for seq_T rows
  __half *d_plain = nullptr;     size_t plain_halfs = 0;   // fp16 models: W^T [out, in]
  __half *d_pscale = nullptr;    size_t pscale_halfs = 0;  // int8: per output row scales, per matrix
  // int8 / int4: every projection a second time in its packed interchange form, row-major (one row per output
  // channel): what the few-row GEMM streams for prompts and for decode of more than 8 streams
  uint8_t *d_qcopy = nullptr;    size_t qcopy_bytes = 0;
  __half *d_qscale = nullptr;    size_t qscale_halfs = 0;
  bool row_copies = true;        // keep the copies the GEMM path needs (FR_B200_ROW_COPIES=0: decode-only model)
  bool rows_planned = false;     // some batch up to max_batch is decoded by the GEMM path
  uint8_t *d_seq = nullptr;      size_t seq_bytes = 0; int seq_T = 0;
  PhaseDev *d_head_phase = nullptr;   // the head as a stand-alone matvec phase
  // greedy runs of many streams: two decode steps captured as a CUDA graph and replayed (the step is ~170 launches)
  GreedyCtl *d_ctl = nullptr;
  uint8_t *d_sample = nullptr; size_t sample_bytes = 0;   // scratch of fr_b200_sample
  uint8_t *d_adj = nullptr; size_t adj_bytes = 0;         // staging of fr_b200_logits_add
  cudaStream_t gstream = nullptr;
  cudaEvent_t gev = nullptr;
  cudaGraphExec_t gexec = nullptr;
  int g_batch = 0; unsigned g_par = 0; const void *g_seq = nullptr;   // what the captured graph was built for
  float *d_lnvec = nullptr;           // ln_out of the last prompt token
  cudaStream_t seq_streams[4] = {nullptr, nullptr, nullptr, nullptr};   // long prompts: one stream per piece of rows
  std::vector<cudaEvent_t> seq_events;                                  // [piece][layer] + one start event
  // scratch for uploads
  void *d_scratch[4] = {nullptr, nullptr, nullptr, nullptr};
  size_t scratch_bytes[4] = {0, 0, 0, 0};
  // bookkeeping
  std::map<std::string, MatrixSlot> mats;
  std::map<std::string, VecSlot> vecs;
  std::vector<char> emb_rows_set;
  bool emb_set = false;
  std::vector<PhaseDev> phases;
  bool finalized = false;
  int n_stages[3] = {0, 0, 0}, grid = 0;   // per decode mode (1, <=4, <=8 streams)
  size_t smem[3] = {0, 0, 0};
  long long launches = 0;
  int l2_prefetch = 384 * 1024;  // bytes per CTA the producer keeps requested from L2 ahead of the ring
  long long stream_bytes = 0;

  int32_t *out_argmax() const { return reinterpret_cast<int32_t *>(d_out + (size_t)cfg.max_batch * Vpad); }
  int *out_status() const { return reinterpret_cast<int *>(out_argmax() + cfg.max_batch); }
  size_t out_bytes() const { return ((size_t)cfg.max_batch * Vpad + cfg.max_batch + 1) * 4; }
};

namespace {

int ensure_scratch(fr_b200_model *m, int idx, size_t bytes) {
  if (m->scratch_bytes[idx] >= bytes) return 0;
  if (m->d_scratch[idx]) cudaFree(m->d_scratch[idx]);
  m->d_scratch[idx] = nullptr;
  m->scratch_bytes[idx] = 0;
  CU(cudaMalloc(&m->d_scratch[idx], bytes));
  m->scratch_bytes[idx] = bytes;
  return 0;
}

void free_scratch(fr_b200_model *m) {
  for (int i = 0; i < 4; ++i) {
    if (m->d_scratch[i]) cudaFree(m->d_scratch[i]);
    m->d_scratch[i] = nullptr;
    m->scratch_bytes[i] = 0;
  }
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Lay out every matrix / vector of the model.  Per layer the weight blob holds the phases in the
// order the kernel streams them.
void plan(fr_b200_model *m) {
  const int C = m->C, F = m->F, fmt = m->fmt;
  size_t woff = 0, roff = 0, voff = 0;
  auto mat = [&](const std::string &name, int K, int N, size_t tile_off, size_t item_stride, size_t rs_off,
                 size_t rs_stride) {
    MatrixSlot s;
    s.K = K; s.N = N; s.tile_off = tile_off; s.item_stride = item_stride; s.rscale_off = rs_off; s.rscale_stride = rs_stride;
    m->mats[name] = s;
  };
  auto vec = [&](const std::string &name, int n) {
    VecSlot s; s.off = voff; s.n = n; voff += (size_t)(n + 7) / 8 * 8;   // 16-byte aligned in the fp16 image too
    m->vecs[name] = s;
  };
  const size_t rbC = rowblock_bytes(fmt, C), rbF = rowblock_bytes(fmt, F);
  const int nbC = C / ROWS, nbF = F / ROWS;
  m->phases.clear();
  int pi = 0;
  auto phase = [&](int kind, int layer, int K, int n_items, int n_sub, size_t w_off, size_t rs_off) {
    PhaseDev p;
    memset(&p, 0, sizeof(p));
    p.w = reinterpret_cast<const uint8_t *>(w_off);        // patched to a pointer in finalize
    p.rscale = reinterpret_cast<const __half *>(rs_off);   // element offset, patched in finalize
    p.kind = kind; p.layer = layer; p.K = K; p.n_items = n_items; p.n_sub = n_sub;
    p.rot = 0;   // set in finalize, once the grid size is known
    ++pi;
    m->phases.push_back(p);
  };
  for (int l = 0; l < m->L; ++l) {
    const std::string b = "blocks." + std::to_string(l) + ".", a = b + "att.", f = b + "ffn.";
    vec(b + "ln1.weight", C); vec(b + "ln1.bias", C); vec(b + "ln2.weight", C); vec(b + "ln2.bias", C);
    vec(a + "time_mix_k", C); vec(a + "time_mix_v", C); vec(a + "time_mix_r", C);
    if (m->gate) vec(a + "time_mix_g", C);
    vec(f + "time_mix_k", C); vec(f + "time_mix_r", C);
    const int nd = m->cfg.version == FR_B200_V5_0 ? m->H : C;
    vec(a + "time_decay", nd); vec(a + "time_first", nd);
    if (m->v5) { vec(a + "ln_x.weight", C); vec(a + "ln_x.bias", C); }
    if (!m->v5) {
      // K,V,R of the same 16 channels sit next to each other: item = [K tile][V tile][R tile]
      mat(a + "key.weight", C, C, woff, 3 * rbC, roff, 3 * ROWS);
      mat(a + "value.weight", C, C, woff + rbC, 3 * rbC, roff + ROWS, 3 * ROWS);
      mat(a + "receptance.weight", C, C, woff + 2 * rbC, 3 * rbC, roff + 2 * ROWS, 3 * ROWS);
      phase(PH_ATT_KVR, l, C, nbC, 3, woff, roff);
      woff += (size_t)nbC * 3 * rbC; roff += (size_t)nbC * 3 * ROWS;
    } else {
      const int ncls = m->gate ? 4 : 3;
      const char *names[4] = {"key.weight", "value.weight", "receptance.weight", "gate.weight"};
      phase(PH5_KVRG, l, C, nbC * ncls, 1, woff, roff);
      for (int c = 0; c < ncls; ++c) {
        mat(a + names[c], C, C, woff, rbC, roff, ROWS);
        woff += (size_t)nbC * rbC; roff += (size_t)nbC * ROWS;
      }
      phase(PH5_WKV, l, 0, 0, 0, 0, 0);
    }
    mat(a + "output.weight", C, C, woff, rbC, roff, ROWS);
    phase(PH_ATT_O, l, C, nbC, 1, woff, roff);
    woff += (size_t)nbC * rbC; roff += (size_t)nbC * ROWS;
    // ffn key rows then ffn receptance rows, both read C inputs
    mat(f + "key.weight", C, F, woff, rbC, roff, ROWS);
    mat(f + "receptance.weight", C, C, woff + (size_t)nbF * rbC, rbC, roff + (size_t)nbF * ROWS, ROWS);
    phase(PH_FFN_KR, l, C, nbF + nbC, 1, woff, roff);
    m->phases.back().split[0] = nbF;
    woff += (size_t)(nbF + nbC) * rbC; roff += (size_t)(nbF + nbC) * ROWS;
    mat(f + "value.weight", F, C, woff, rbF, roff, ROWS);
    phase(PH_FFN_V, l, F, nbC, 1, woff, roff);
    woff += (size_t)nbC * rbF; roff += (size_t)nbC * ROWS;
  }
  vec("ln_out.weight", C); vec("ln_out.bias", C);
  const int nbV = m->Vpad / ROWS;
  mat("head.weight", C, m->V, woff, rbC, roff, ROWS);
  phase(PH_HEAD, 0, C, nbV, 1, woff, roff);
  woff += (size_t)nbV * rbC; roff += (size_t)nbV * ROWS;
  m->weights_bytes = woff; m->rscale_n = roff; m->vecs_n = voff;
  m->plain_halfs = 0; m->pscale_halfs = 0; m->qcopy_bytes = 0; m->qscale_halfs = 0;
  // The GEMM path (prompts, and decode of more than 8 streams at once) reads the projections row by output channel:
  // fp16 models keep W^T fp16 [N, K] (with the head when more than 8 streams can be decoded: all rows want logits;
  // a prompt's head is a matvec over the last token), made at load for RWKV-5.x and for max_batch > 8, else on the
  // first long prompt; int8 / int4 models keep the packed codes row-major [N, K] / [N, K/2] (+ scales), the same
  // bytes as the streaming tiles, which the GEMM expands in shared memory.
  // (also when the persistent kernel cannot carry max_batch streams of a model this wide: its shared memory holds the
  // activation vectors of every stream, e.g. 8 streams x 8192 channel-mix inputs do not fit)
  bool big = m->cfg.max_batch > MAX_B;
  if (!big) {
    int optin = 0;
    if (cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, m->device) == cudaSuccess)
      for (int mode = 1; mode <= decode_mode(m->cfg.max_batch); ++mode)
        if (decode_smem_bytes(fmt, mode, C, F, m->v5 ? 5 : 4, 2, 1) > (size_t)optin) big = true;
  }
  m->rows_planned = big;
  for (auto &kv : m->mats) {
    MatrixSlot &ms = kv.second;
    if (fmt == FMT_FP16) {
      if (kv.first == "head.weight" && !big) continue;
      ms.has_plain = true;
      ms.plain_off = m->plain_halfs;
      m->plain_halfs += ((size_t)ms.K * ms.N + 127) / 128 * 128;
    } else if (m->row_copies) {
      ms.q_off = m->qcopy_bytes;
      m->qcopy_bytes += ((size_t)ms.N * (fmt == FMT_INT8 ? ms.K : ms.K / 2) + 255) / 256 * 256;
      ms.pscale_off = m->pscale_halfs;
      if (fmt == FMT_INT8) m->pscale_halfs += ((size_t)ms.N + 7) / 8 * 8;
      ms.qs_off = m->qscale_halfs;
      if (fmt == FMT_INT4) m->qscale_halfs += ((size_t)ms.N * (ms.K / 32) + 7) / 8 * 8;
    }
  }
  m->stream_bytes = (long long)woff + (fmt == FMT_INT8 ? (long long)roff * 2 : 0);
}

bool is_host_ptr(const void *p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return true; }
  return a.type == cudaMemoryTypeUnregistered || a.type == cudaMemoryTypeHost;
}

int upload_matrix(fr_b200_model *m, const MatrixSlot &s, const void *data, int dtype) {
  const size_t n = (size_t)s.K * s.N;
  const size_t in_bytes = n * (dtype == FR_B200_T_F16 ? 2 : 4);
  int rc;
  if ((rc = ensure_scratch(m, 0, in_bytes))) return rc;
  CU(cudaMemcpy(m->d_scratch[0], data, in_bytes, cudaMemcpyDefault));
  uint8_t *dst = m->d_weights + s.tile_off;
  if (m->fmt == FMT_FP16) {
    const __half *src = reinterpret_cast<const __half *>(m->d_scratch[0]);
    if (dtype == FR_B200_T_F32) {
      if ((rc = ensure_scratch(m, 1, n * 2))) return rc;
      CU(launch_f32_to_f16(reinterpret_cast<const float *>(m->d_scratch[0]), reinterpret_cast<__half *>(m->d_scratch[1]), n, 0));
      src = reinterpret_cast<const __half *>(m->d_scratch[1]);
    }
    CU(launch_pack(FMT_FP16, src, nullptr, s.K, s.N, dst, s.item_stride, nullptr, 0, 0));
    if (s.has_plain && m->d_plain) CU(launch_transpose_f16(src, s.K, s.N, m->d_plain + s.plain_off, 0));
  } else {
    const float *w32 = reinterpret_cast<const float *>(m->d_scratch[0]);
    if (dtype == FR_B200_T_F16) {
      if ((rc = ensure_scratch(m, 1, n * 4))) return rc;
      CU(launch_f16_to_f32(reinterpret_cast<const __half *>(m->d_scratch[0]), reinterpret_cast<float *>(m->d_scratch[1]), n, 0));
      w32 = reinterpret_cast<const float *>(m->d_scratch[1]);
    }
    if (m->fmt == FMT_INT8) {
      if ((rc = ensure_scratch(m, 2, n))) return rc;
      if ((rc = ensure_scratch(m, 3, (size_t)s.N * 2))) return rc;
      CU(launch_quant_int8(w32, s.K, s.N, reinterpret_cast<int8_t *>(m->d_scratch[2]), reinterpret_cast<__half *>(m->d_scratch[3]), 0));
      CU(launch_pack(FMT_INT8, m->d_scratch[2], reinterpret_cast<const __half *>(m->d_scratch[3]), s.K, s.N, dst,
                     s.item_stride, m->d_rscale + s.rscale_off, s.rscale_stride, 0));
      if (m->d_qcopy) {
        // the codes are [N, K] already; the row scale is applied to the GEMM's accumulator
        CU(cudaMemcpy(m->d_qcopy + s.q_off, m->d_scratch[2], n, cudaMemcpyDeviceToDevice));
        CU(cudaMemcpy(m->d_pscale + s.pscale_off, m->d_scratch[3], (size_t)s.N * 2, cudaMemcpyDeviceToDevice));
      }
    } else {
      if ((rc = ensure_scratch(m, 2, n / 2))) return rc;
      if ((rc = ensure_scratch(m, 3, (size_t)s.N * (s.K / 32) * 2))) return rc;
      CU(launch_quant_int4(w32, s.K, s.N, reinterpret_cast<uint8_t *>(m->d_scratch[2]), reinterpret_cast<__half *>(m->d_scratch[3]), 0));
      CU(launch_pack(FMT_INT4, m->d_scratch[2], reinterpret_cast<const __half *>(m->d_scratch[3]), s.K, s.N, dst,
                     s.item_stride, nullptr, 0, 0));
      if (m->d_qcopy) {
        CU(cudaMemcpy(m->d_qcopy + s.q_off, m->d_scratch[2], n / 2, cudaMemcpyDeviceToDevice));
        CU(cudaMemcpy(m->d_qscale + s.qs_off, m->d_scratch[3], (size_t)s.N * (s.K / 32) * 2, cudaMemcpyDeviceToDevice));
      }
    }
  }
  CU(cudaDeviceSynchronize());
  return 0;
}

// small tensors: bring to host, convert to fp32
int to_host_f32(const void *data, int dtype, size_t n, std::vector<float> &out) {
  out.resize(n);
  if (dtype == FR_B200_T_F32) {
    CU(cudaMemcpy(out.data(), data, n * 4, cudaMemcpyDefault));
  } else {
    std::vector<__half> tmp(n);
    CU(cudaMemcpy(tmp.data(), data, n * 2, cudaMemcpyDefault));
    for (size_t i = 0; i < n; ++i) out[i] = __half2float(tmp[i]);
  }
  return 0;
}

int check_status(fr_b200_model *m, int st) {
  if (st == 0) return 0;
  // a bounded wait gave up: clear the status word for the next launch
  cudaMemset(m->out_status(), 0, 4);
  m->exch_batch = 0;   // exchange vectors may be half written
  return fail(FR_B200_E_TIMEOUT, "device-side wait timed out (code " + std::to_string(st) + ")");
}

}  // namespace

namespace {
struct DevBuf {
  void *p = nullptr;
  ~DevBuf() { if (p) cudaFree(p); }
  cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 256); }
};
}  // namespace

extern "C" {

const char *fr_b200_strerror(int status) {
  switch (status) {
    case FR_B200_OK: return "ok";
    case FR_B200_E_ARG: return "bad argument";
    case FR_B200_E_UNSUPPORTED: return "unsupported model shape, version or batch";
    case FR_B200_E_CUDA: return "CUDA runtime error";
    case FR_B200_E_STATE: return "call order violation";
    case FR_B200_E_MISSING: return "model tensor missing at finalize";
    case FR_B200_E_TIMEOUT: return "device-side wait timed out";
    case FR_B200_E_NOMEM: return "out of memory";
    default: return "unknown status";
  }
}
const char *fr_b200_last_error(void) { return g_err.c_str(); }

int fr_b200_create(const fr_b200_config *cfg, fr_b200_model **out) {
  if (!cfg || !out) return fail(FR_B200_E_ARG, "null argument");
  *out = nullptr;
  const int v = cfg->version;
  if (v != FR_B200_V4 && v != FR_B200_V5_0 && v != FR_B200_V5_1 && v != FR_B200_V5_2)
    return fail(FR_B200_E_UNSUPPORTED, "version must be 4, 50, 51 or 52");
  if (cfg->n_layer <= 0 || cfg->vocab <= 0) return fail(FR_B200_E_ARG, "n_layer and vocab must be positive");
  if (cfg->n_embd <= 0 || cfg->n_embd % 64 || cfg->n_ffn <= 0 || cfg->n_ffn % 64)
    return fail(FR_B200_E_UNSUPPORTED, "n_embd and n_ffn must be positive multiples of 64");
  if (cfg->weight_format < 0 || cfg->weight_format > 2) return fail(FR_B200_E_ARG, "bad weight_format");
  if (cfg->max_batch < 1 || cfg->max_batch > 4096) return fail(FR_B200_E_UNSUPPORTED, "max_batch must be 1..4096");
  if (v != FR_B200_V4 && (cfg->n_head <= 0 || cfg->n_embd != cfg->n_head * 64))
    return fail(FR_B200_E_UNSUPPORTED, "RWKV-5 needs n_embd == 64 * n_head");
  int ndev = 0;
  CU(cudaGetDeviceCount(&ndev));
  if (cfg->device < 0 || cfg->device >= ndev) return fail(FR_B200_E_ARG, "no such CUDA device");
  CU(cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  CU(cudaGetDeviceProperties(&prop, cfg->device));
  if (prop.major != 10) return fail(FR_B200_E_UNSUPPORTED, "this library is built for sm_100a (B200) only");

  fr_b200_model *m = new (std::nothrow) fr_b200_model();
  if (!m) return fail(FR_B200_E_NOMEM, "host allocation failed");
  m->cfg = *cfg;
  m->C = cfg->n_embd; m->F = cfg->n_ffn; m->V = cfg->vocab; m->L = cfg->n_layer; m->H = cfg->n_head;
  m->Vpad = (cfg->vocab + ROWS - 1) / ROWS * ROWS;
  m->fmt = cfg->weight_format;
  m->v5 = v != FR_B200_V4;
  m->gate = v == FR_B200_V5_1 || v == FR_B200_V5_2;
  m->device = cfg->device;
  m->par.assign(cfg->max_batch, 0u);
  if (const char *e = getenv("FR_B200_ROW_COPIES")) m->row_copies = atoi(e) != 0;
  if ((m->C + prop.multiProcessorCount - 1) / prop.multiProcessorCount > 128) {
    delete m;
    return fail(FR_B200_E_UNSUPPORTED, "n_embd too large for the shift-state stash");
  }
  plan(m);
  m->layer_stride = layer_bytes(m->C, m->H, m->v5, cfg->act_fp16);
  m->state_stride = align256(m->layer_stride * m->L);
  const int B = cfg->max_batch;
  auto alloc = [&](void **p, size_t bytes) -> int {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 256);
    if (e != cudaSuccess) return fail(e == cudaErrorMemoryAllocation ? FR_B200_E_NOMEM : FR_B200_E_CUDA,
                                      std::string("cudaMalloc: ") + cudaGetErrorString(e));
    return 0;
  };
  int rc = 0;
  if (!rc) rc = alloc((void **)&m->d_weights, m->weights_bytes);
  if (!rc) rc = alloc((void **)&m->d_rscale, m->rscale_n * 2);
  if (!rc) rc = alloc((void **)&m->d_vecs, m->vecs_n * 4);
  if (!rc && cfg->host_visible_state) {
    // managed memory, resident on the device: the host may read it between calls (a page then migrates and comes back
    // with the next launch)
    cudaError_t e = cudaMallocManaged((void **)&m->d_state, m->state_stride * B);
    if (e != cudaSuccess) rc = fail(FR_B200_E_NOMEM, std::string("cudaMallocManaged(state): ") + cudaGetErrorString(e));
    else {
      cudaMemLocation loc;
      loc.type = cudaMemLocationTypeDevice; loc.id = cfg->device;
      cudaMemAdvise(m->d_state, m->state_stride * B, cudaMemAdviseSetPreferredLocation, loc);
      cudaGetLastError();   // the advice is an optimisation: a platform that refuses it still works
    }
  } else if (!rc) rc = alloc((void **)&m->d_state, m->state_stride * B);
  if (!rc) rc = alloc((void **)&m->d_x, (size_t)B * m->C * sizeof(exch_t));
  if (!rc) rc = alloc((void **)&m->d_xa, (size_t)B * m->C * sizeof(exch_t));
  if (!rc) rc = alloc((void **)&m->d_rwkv, (size_t)B * m->C * sizeof(exch_t));
  if (!rc) rc = alloc((void **)&m->d_kk, (size_t)B * m->F * sizeof(exch_t));
  if (!rc) rc = alloc((void **)&m->d_rr, (size_t)B * m->C * sizeof(exch_t));
  if (!rc) rc = alloc((void **)&m->d_v5buf, (size_t)5 * B * m->C * sizeof(exch_t));
  if (!rc) rc = alloc((void **)&m->d_out, m->out_bytes());
  if (!rc) rc = alloc((void **)&m->d_amax, (size_t)B * 8);
  // fp16 W^T copies now for RWKV-5.x (seq kernels) and for models that decode more than 8 streams; else on demand
  if (!rc && m->plain_halfs && m->row_copies && (m->v5 || m->rows_planned)) rc = alloc((void **)&m->d_plain, m->plain_halfs * 2);
  if (!rc && m->qcopy_bytes) rc = alloc((void **)&m->d_qcopy, m->qcopy_bytes);
  if (!rc && m->qscale_halfs) rc = alloc((void **)&m->d_qscale, m->qscale_halfs * 2);
  if (!rc && m->pscale_halfs) rc = alloc((void **)&m->d_pscale, m->pscale_halfs * 2);
  if (!rc) rc = alloc((void **)&m->d_head_phase, sizeof(PhaseDev));
  if (!rc) rc = alloc((void **)&m->d_ctl, sizeof(GreedyCtl));
  if (!rc) rc = alloc((void **)&m->d_lnvec, (size_t)m->C * 4);
  if (!rc) rc = alloc((void **)&m->d_layers, sizeof(LayerDev) * m->L);
  if (!rc) rc = alloc((void **)&m->d_phases, sizeof(PhaseDev) * m->phases.size());
  if (!rc && cudaMallocHost((void **)&m->h_out, m->out_bytes()) != cudaSuccess) rc = fail(FR_B200_E_NOMEM, "cudaMallocHost failed");
  if (rc) { fr_b200_destroy(m); return rc; }
  cudaMemset(m->d_weights, 0, m->weights_bytes);
  cudaMemset(m->d_rscale, 0, m->rscale_n * 2);
  cudaMemset(m->d_out, 0, m->out_bytes());
  // tag 0 is never expected by a reader
  m->exch_batch = 0;   // the first launch clears the exchange vectors
  m->emb_rows_set.assign(m->V, 0);
  *out = m;
  return FR_B200_OK;
}

void fr_b200_destroy(fr_b200_model *m) {
  if (!m) return;
  cudaSetDevice(m->device);
  free_scratch(m);
  void *ptrs[] = {m->d_weights, m->d_rscale, m->d_vecs, m->d_vecs16, m->d_emb, m->d_state, m->d_x, m->d_xa, m->d_rwkv, m->d_kk, m->d_rr,
                  m->d_v5buf, m->d_out, m->d_layers, m->d_phases, m->d_amax, m->d_plain, m->d_pscale, m->d_qcopy, m->d_qscale, m->d_seq, m->d_head_phase, m->d_lnvec};
  for (void *p : ptrs)
    if (p) cudaFree(p);
  if (m->h_out) cudaFreeHost(m->h_out);
  if (m->gexec) cudaGraphExecDestroy(m->gexec);
  if (m->gev) cudaEventDestroy(m->gev);
  if (m->gstream) cudaStreamDestroy(m->gstream);
  for (cudaEvent_t ev : m->seq_events) cudaEventDestroy(ev);
  for (cudaStream_t sq : m->seq_streams) if (sq) cudaStreamDestroy(sq);
  if (m->d_ctl) cudaFree(m->d_ctl);
  if (m->d_sample) cudaFree(m->d_sample);
  if (m->d_adj) cudaFree(m->d_adj);
  if (m->d_hist) cudaFree(m->d_hist);
  delete m;
}

int fr_b200_set_tensor(fr_b200_model *m, const char *name, const void *data, int dtype, const int64_t *shape, int ndim) {
  if (!m || !name || !data || (ndim > 0 && !shape)) return fail(FR_B200_E_ARG, "null argument");
  if (dtype != FR_B200_T_F16 && dtype != FR_B200_T_F32) return fail(FR_B200_E_ARG, "dtype must be f16 or f32");
  if (m->finalized) return fail(FR_B200_E_STATE, "model already finalized");
  CU(cudaSetDevice(m->device));
  size_t numel = 1;
  for (int i = 0; i < ndim; ++i) {
    if (shape[i] <= 0) return fail(FR_B200_E_ARG, "non-positive dimension");
    numel *= (size_t)shape[i];
  }
  const std::string nm(name);
  if (nm == "emb.weight" || nm.rfind("emb.", 0) == 0 || nm.rfind("embd_", 0) == 0) {
    size_t row0 = 0, rows = 0;
    if (nm == "emb.weight") {
      if (ndim != 2 || shape[0] != m->V || shape[1] != m->C) return fail(FR_B200_E_ARG, "emb.weight must be [vocab, n_embd]");
      rows = m->V;
    } else {
      const char *num = nm.c_str() + (nm[3] == '.' ? 4 : 5);
      char *end = nullptr;
      long r = strtol(num, &end, 10);
      if (end == num || *end || r < 0 || r >= m->V) return fail(FR_B200_E_ARG, "bad embedding row name " + nm);
      if (numel != (size_t)m->C) return fail(FR_B200_E_ARG, "embedding row must have n_embd elements");
      row0 = (size_t)r; rows = 1;
    }
    if (m->emb_dtype < 0) {
      m->emb_dtype = dtype;
      cudaError_t e = cudaMalloc((void **)&m->d_emb, (size_t)m->V * m->C * (dtype == FR_B200_T_F16 ? 2 : 4));
      if (e != cudaSuccess) return fail(FR_B200_E_NOMEM, std::string("cudaMalloc(emb): ") + cudaGetErrorString(e));
    } else if (m->emb_dtype != dtype) {
      return fail(FR_B200_E_ARG, "embedding rows must all have the same dtype");
    }
    const size_t es = dtype == FR_B200_T_F16 ? 2 : 4;
    CU(cudaMemcpy(m->d_emb + row0 * m->C * es, data, rows * m->C * es, cudaMemcpyDefault));
    for (size_t r = row0; r < row0 + rows; ++r) m->emb_rows_set[r] = 1;
    return FR_B200_OK;
  }
  auto mi = m->mats.find(nm);
  if (mi != m->mats.end()) {
    MatrixSlot &s = mi->second;
    if (ndim != 2 || shape[0] != s.K || shape[1] != s.N)
      return fail(FR_B200_E_ARG, nm + ": expected [" + std::to_string(s.K) + ", " + std::to_string(s.N) + "] (in, out)");
    int rc = upload_matrix(m, s, data, dtype);
    if (rc) return rc;
    s.set = true;
    return FR_B200_OK;
  }
  auto vi = m->vecs.find(nm);
  if (vi != m->vecs.end()) {
    VecSlot &s = vi->second;
    if (numel != (size_t)s.n) return fail(FR_B200_E_ARG, nm + ": expected " + std::to_string(s.n) + " elements");
    std::vector<float> h;
    int rc = to_host_f32(data, dtype, numel, h);
    if (rc) return rc;
    CU(cudaMemcpy(m->d_vecs + s.off, h.data(), numel * 4, cudaMemcpyHostToDevice));
    s.set = true;
    return FR_B200_OK;
  }
  return fail(FR_B200_E_ARG, "unknown tensor name " + nm);
}

int fr_b200_finalize(fr_b200_model *m) {
  if (!m) return fail(FR_B200_E_ARG, "null model");
  if (m->finalized) return FR_B200_OK;
  CU(cudaSetDevice(m->device));
  for (auto &kv : m->mats) if (!kv.second.set) return fail(FR_B200_E_MISSING, "missing tensor " + kv.first);
  for (auto &kv : m->vecs) if (!kv.second.set) return fail(FR_B200_E_MISSING, "missing tensor " + kv.first);
  for (int r = 0; r < m->V; ++r) if (!m->emb_rows_set[r]) return fail(FR_B200_E_MISSING, "missing embedding row " + std::to_string(r));
  free_scratch(m);
  // layer table
  std::vector<LayerDev> layers(m->L);
  auto vp = [&](const std::string &n) -> const float * { return m->d_vecs + m->vecs[n].off; };
  for (int l = 0; l < m->L; ++l) {
    const std::string b = "blocks." + std::to_string(l) + ".", a = b + "att.", f = b + "ffn.";
    LayerDev &d = layers[l];
    memset(&d, 0, sizeof(d));
    d.ln1_w = vp(b + "ln1.weight"); d.ln1_b = vp(b + "ln1.bias"); d.ln2_w = vp(b + "ln2.weight"); d.ln2_b = vp(b + "ln2.bias");
    d.att_mix[0] = vp(a + "time_mix_k"); d.att_mix[1] = vp(a + "time_mix_v"); d.att_mix[2] = vp(a + "time_mix_r");
    d.att_mix[3] = m->gate ? vp(a + "time_mix_g") : nullptr;
    d.ffn_mix[0] = vp(f + "time_mix_k"); d.ffn_mix[1] = vp(f + "time_mix_r");
    d.decay = vp(a + "time_decay"); d.first = vp(a + "time_first");
    if (m->v5) { d.lnx_w = vp(a + "ln_x.weight"); d.lnx_b = vp(a + "ln_x.bias"); }
  }
  CU(cudaMemcpy(m->d_layers, layers.data(), sizeof(LayerDev) * m->L, cudaMemcpyHostToDevice));
  // LayerNorm weights / biases and the mix vectors as fp16, when that loses nothing (files of the fp16 strategy):
  // the one-stream kernel stages them in half the shared memory
  bool par16 = m->cfg.act_fp16 != 0;
  if (const char *e = getenv("FR_B200_PAR16")) par16 = par16 && atoi(e) != 0;
  if (par16) {
    std::vector<float> hv(m->vecs_n);
    CU(cudaMemcpy(hv.data(), m->d_vecs, m->vecs_n * 4, cudaMemcpyDeviceToHost));
    std::vector<__half> h16(m->vecs_n);
    for (auto &kv : m->vecs) {
      const std::string &n = kv.first;
      const bool staged = n.find("ln1.") != std::string::npos || n.find("ln2.") != std::string::npos ||
                          n.find("time_mix_") != std::string::npos || n.rfind("ln_out.", 0) == 0;
      for (int i = 0; i < kv.second.n; ++i) {
        const float f = hv[kv.second.off + i];
        const __half h = __float2half_rn(f);
        h16[kv.second.off + i] = h;
        if (staged && __half2float(h) != f) par16 = false;
      }
    }
    if (par16) {
      CU(cudaMalloc((void **)&m->d_vecs16, m->vecs_n * 2));
      CU(cudaMemcpy(m->d_vecs16, h16.data(), m->vecs_n * 2, cudaMemcpyHostToDevice));
    }
  }
  // kernel geometry: as many ring stages as shared memory allows (capped), one CTA per SM
  int optin = 0;
  CU(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, m->device));
  int want = MAX_STAGES;
  if (const char *e = getenv("FR_B200_STAGES")) want = atoi(e);
  if (const char *e = getenv("FR_B200_L2_PREFETCH_KB")) m->l2_prefetch = atoi(e) * 1024;
  if (want < 2) want = 2;
  if (want > MAX_STAGES) want = MAX_STAGES;
  const int ver = m->v5 ? 5 : 4;
  const int max_mode = decode_mode(std::min(m->cfg.max_batch, MAX_B));
  for (int mode = 0; mode <= max_mode; ++mode) {
    int st = 0;
    for (int s = want; s >= 2; --s)
      if (decode_smem_bytes(m->fmt, mode, m->C, m->F, ver, s, m->d_vecs16 != nullptr) <= (size_t)optin) { st = s; break; }
    if (st == 0) {
      if (m->rows_planned && mode > 0) { m->n_stages[mode] = 0; continue; }   // such batches take the GEMM path
      return fail(FR_B200_E_UNSUPPORTED, "model too wide for shared memory at this batch size (max_batch " +
                                             std::to_string(m->cfg.max_batch) + ")");
    }
    m->n_stages[mode] = st;
    m->smem[mode] = decode_smem_bytes(m->fmt, mode, m->C, m->F, ver, st, m->d_vecs16 != nullptr);
    int g = 0;
    CU(decode_max_grid(m->fmt, mode, m->smem[mode], m->device, &g));
    if (g == 0) return fail(FR_B200_E_UNSUPPORTED, "decode kernel does not fit on an SM");
    m->grid = g;
  }
  // stash capacity: ceil(C / grid) channels per CTA
  if ((m->C + m->grid - 1) / m->grid > 128) return fail(FR_B200_E_UNSUPPORTED, "n_embd too large for the shift-state stash");
  // phase table with real pointers; rotate item ownership from phase to phase
  std::vector<PhaseDev> ph = m->phases;
  for (size_t i = 0; i < ph.size(); ++i) {
    ph[i].w = m->d_weights + reinterpret_cast<size_t>(ph[i].w);
    ph[i].rscale = m->fmt == FMT_INT8 ? m->d_rscale + reinterpret_cast<size_t>(ph[i].rscale) : nullptr;
    ph[i].rot = (int)((i * 37) % (size_t)m->grid);
    if (ph[i].kind == PH_ATT_KVR || ph[i].kind == PH5_WKV) { ph[i].aux0 = layers[ph[i].layer].first; ph[i].aux1 = layers[ph[i].layer].decay; }
    if (ph[i].kind == PH_ATT_O && m->v5) { ph[i].aux0 = layers[ph[i].layer].lnx_w; ph[i].aux1 = layers[ph[i].layer].lnx_b; }
  }
  CU(cudaMemcpy(m->d_phases, ph.data(), sizeof(PhaseDev) * ph.size(), cudaMemcpyHostToDevice));
  {
    PhaseDev hp = ph.back();   // the head, as the one phase of a stand-alone matvec launch
    hp.kind = PH_MATVEC; hp.rot = 0;
    CU(cudaMemcpy(m->d_head_phase, &hp, sizeof(hp), cudaMemcpyHostToDevice));
  }
  m->finalized = true;
  return fr_b200_state_reset(m, -1);
}

namespace {
// Streams that are decoded together read the same copy of their token-shift states (the kernels take one parity per
// launch).  A stream that was reset, imported or prefilled on its own may be one token out of step with stream 0:
// its current copy is duplicated into the other one and its parity flipped, which changes nothing it will read.
int align_parity(fr_b200_model *m, int batch, cudaStream_t st) {
  const size_t ab = act_bytes(m->cfg.act_fp16), row = (size_t)m->C * ab;
  for (int b = 1; b < batch; ++b) {
    if (m->par[b] == m->par[0]) continue;
    const int par = (int)m->par[b];
    uint8_t *base = m->d_state + (size_t)b * m->state_stride;
    CU(cudaMemcpy2DAsync(base + off_sx(m->C, m->cfg.act_fp16, par ^ 1), m->layer_stride, base + off_sx(m->C, m->cfg.act_fp16, par),
                         m->layer_stride, row, m->L, cudaMemcpyDeviceToDevice, st));
    CU(cudaMemcpy2DAsync(base + off_ffn_sx(m->C, m->H, m->v5, m->cfg.act_fp16, par ^ 1), m->layer_stride,
                         base + off_ffn_sx(m->C, m->H, m->v5, m->cfg.act_fp16, par), m->layer_stride, row, m->L,
                         cudaMemcpyDeviceToDevice, st));
    m->par[b] ^= 1u;
  }
  return 0;
}
int rows_forward(fr_b200_model *m, bool batch_mode, int slot, const int32_t *ids, int R, cudaStream_t st);
// more streams than the persistent kernel carries (or a model too wide for that many): the GEMM path decodes them
bool decode_by_rows(const fr_b200_model *m, int batch) { return batch > MAX_B || m->n_stages[decode_mode(batch)] == 0; }
// fp16 models that were created without the W^T copies build them from the streaming tiles (exact: the tiles hold
// the same fp16 values) the first time the GEMM path is asked for
int ensure_row_copies(fr_b200_model *m) {
  if (m->d_plain || m->d_qcopy) return 0;
  if (m->fmt != FMT_FP16 || !m->row_copies || !m->plain_halfs) return fail(FR_B200_E_UNSUPPORTED, "the model keeps no row copies for the GEMM path");
  CU(cudaDeviceSynchronize());
  cudaError_t e = cudaMalloc((void **)&m->d_plain, m->plain_halfs * 2);
  if (e != cudaSuccess) { m->d_plain = nullptr; return fail(FR_B200_E_NOMEM, std::string("cudaMalloc(row copies): ") + cudaGetErrorString(e)); }
  for (auto &kv : m->mats) {
    const MatrixSlot &s = kv.second;
    if (!s.has_plain) continue;
    const size_t n = (size_t)s.K * s.N;
    int rc;
    if ((rc = ensure_scratch(m, 0, n * 4))) return rc;
    if ((rc = ensure_scratch(m, 1, n * 2))) return rc;
    CU(launch_unpack(FMT_FP16, m->d_weights + s.tile_off, s.item_stride, nullptr, 0, s.K, s.N, reinterpret_cast<float *>(m->d_scratch[0]), 0));
    CU(launch_f32_to_f16(reinterpret_cast<const float *>(m->d_scratch[0]), reinterpret_cast<__half *>(m->d_scratch[1]), n, 0));
    CU(launch_transpose_f16(reinterpret_cast<const __half *>(m->d_scratch[1]), s.K, s.N, m->d_plain + s.plain_off, 0));
  }
  CU(cudaDeviceSynchronize());
  free_scratch(m);
  return 0;
}
bool rows_path_built(const fr_b200_model *m) { return m->d_plain || m->d_qcopy; }
int rows_decode_check(fr_b200_model *m, const int32_t *ids_host, int batch, cudaStream_t st) {
  if (m->fmt == FMT_FP16 && !m->mats["head.weight"].has_plain)
    return fail(FR_B200_E_UNSUPPORTED, "this batch size needs the GEMM path, which the model was created without");
  {
    int rc = ensure_row_copies(m);
    if (rc) return rc;
  }
  for (int b = 0; b < batch; ++b)
    if (ids_host && (ids_host[b] < 0 || ids_host[b] >= m->V)) return fail(FR_B200_E_ARG, "token id out of range");
  return align_parity(m, batch, st);
}
}  // namespace

static int decode_impl(fr_b200_model *m, const int32_t *ids_host, const unsigned long long *ids_packed, int batch,
                       cudaStream_t st, unsigned long long *amax, unsigned long long *prof = nullptr) {
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.version = m->cfg.version == FR_B200_V4 ? 4 : m->cfg.version;
  p.L = m->L; p.C = m->C; p.F = m->F; p.V = m->V; p.Vpad = m->Vpad; p.H = m->H;
  p.fmt = m->fmt; p.act_fp16 = m->cfg.act_fp16; p.rescale_every = m->cfg.act_fp16 ? 6 : 0;
  p.B = batch;
  p.n_phases = (int)m->phases.size();
  const int mode = decode_mode(batch);
  const size_t smem = m->smem[mode];
  p.n_stages = m->n_stages[mode];
  if (ids_host)
    for (int b = 0; b < batch; ++b) {
      if (ids_host[b] < 0 || ids_host[b] >= m->V) return fail(FR_B200_E_ARG, "token id out of range");
      p.ids_val[b] = ids_host[b];
    }
  p.ids_packed = ids_packed;
  p.amax = amax;
  p.emb = m->d_emb; p.emb_f32 = m->emb_dtype == FR_B200_T_F32; p.layers = m->d_layers; p.phases = m->d_phases;
  p.lnout_w = m->d_vecs + m->vecs["ln_out.weight"].off;
  p.lnout_b = m->d_vecs + m->vecs["ln_out.bias"].off;
  p.vecs16 = m->d_vecs16; p.vecs32 = m->d_vecs;
  p.x = m->d_x; p.xa = m->d_xa; p.rwkv = m->d_rwkv; p.kk = m->d_kk; p.rr = m->d_rr; p.logits = m->d_out;
  // Exchange words carry 8-bit tags: unambiguous only against the write just before them in the same slot.  Slots of
  // streams the previous launch did not write, or words a failed launch left half written, could alias: start clean.
  if (m->exch_batch != batch) {
    const size_t B = m->cfg.max_batch;
    CU(cudaMemsetAsync(m->d_x, 0, B * m->C * sizeof(exch_t), st));
    CU(cudaMemsetAsync(m->d_xa, 0, B * m->C * sizeof(exch_t), st));
    CU(cudaMemsetAsync(m->d_rwkv, 0, B * m->C * sizeof(exch_t), st));
    CU(cudaMemsetAsync(m->d_kk, 0, B * m->F * sizeof(exch_t), st));
    CU(cudaMemsetAsync(m->d_rr, 0, B * m->C * sizeof(exch_t), st));
    CU(cudaMemsetAsync(m->d_v5buf, 0, 5 * B * m->C * sizeof(exch_t), st));
    m->exch_batch = batch;
  }
  p.seq_base = 255u + m->seq;
  {
    int rc = align_parity(m, batch, st);
    if (rc) return rc;
  }
  p.par_mask = 0;
  for (int b = 0; b < batch; ++b) p.par_mask |= m->par[b] << b;
  const size_t bc = (size_t)m->cfg.max_batch * m->C;
  p.k5 = m->d_v5buf; p.v5 = p.k5 + bc; p.r5 = p.v5 + bc; p.g5 = p.r5 + bc; p.o5 = p.g5 + bc;
  p.state = m->d_state; p.state_stride = m->state_stride; p.layer_stride = m->layer_stride;
  p.status = m->out_status();
  p.prof = prof;
  p.l2_prefetch_bytes = m->l2_prefetch;
  CU(launch_decode(p, mode, m->grid, smem, st));
  m->launches++;
  // a phase count that is a multiple of 255 would give consecutive tokens identical tags: skip one tag per token then
  m->seq = (m->seq + (unsigned)m->phases.size() + (m->phases.size() % 255u == 0 ? 1u : 0u)) % 255u;
  for (int b = 0; b < batch; ++b) m->par[b] ^= 1u;
  return 0;
}

int fr_b200_decode(fr_b200_model *m, const int32_t *ids, int batch, float *logits, int32_t *argmax, void *stream) {
  if (!m || !ids) return fail(FR_B200_E_ARG, "null argument");
  if (!m->finalized) return fail(FR_B200_E_STATE, "finalize the model first");
  if (batch < 1 || batch > m->cfg.max_batch) return fail(FR_B200_E_ARG, "batch must be 1..max_batch");
  CU(cudaSetDevice(m->device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  if (decode_by_rows(m, batch)) {
    if ((rc = rows_decode_check(m, ids, batch, st))) return rc;
    if ((rc = rows_forward(m, true, 0, ids, batch, st))) return rc;
    if (argmax) {
      CU(launch_argmax_rows(m->d_out, batch, m->V, m->Vpad, m->out_argmax(), nullptr, st));
      m->launches++;
    }
  } else {
    if (argmax) CU(cudaMemsetAsync(m->d_amax, 0, (size_t)batch * 8, st));
    rc = decode_impl(m, ids, nullptr, batch, st, argmax ? m->d_amax : nullptr);
    if (rc) return rc;
    if (argmax) {
      CU(launch_unpack_ids(m->d_amax, batch, m->out_argmax(), st));
      m->launches++;
    }
  }
  const bool lh = logits && is_host_ptr(logits), ah = argmax && is_host_ptr(argmax);
  if (logits && !lh)
    CU(cudaMemcpy2DAsync(logits, (size_t)m->V * 4, m->d_out, (size_t)m->Vpad * 4, (size_t)m->V * 4, batch, cudaMemcpyDeviceToDevice, st));
  if (argmax && !ah) CU(cudaMemcpyAsync(argmax, m->out_argmax(), (size_t)batch * 4, cudaMemcpyDeviceToDevice, st));
  if (lh || ah) {
    // one D2H of [logits rows used][argmax][status] into the pinned mirror, then hand out
    const size_t tail_off = (size_t)m->cfg.max_batch * m->Vpad * 4;
    if (lh) CU(cudaMemcpyAsync(m->h_out, m->d_out, (size_t)batch * m->Vpad * 4, cudaMemcpyDeviceToHost, st));
    CU(cudaMemcpyAsync(m->h_out + tail_off, reinterpret_cast<uint8_t *>(m->d_out) + tail_off, (size_t)(m->cfg.max_batch + 1) * 4,
                       cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    const int status = *reinterpret_cast<int *>(m->h_out + tail_off + (size_t)m->cfg.max_batch * 4);
    if ((rc = check_status(m, status))) return rc;
    if (lh)
      for (int b = 0; b < batch; ++b)
        memcpy(logits + (size_t)b * m->V, m->h_out + (size_t)b * m->Vpad * 4, (size_t)m->V * 4);
    if (ah) memcpy(argmax, m->h_out + tail_off, (size_t)batch * 4);
  }
  return FR_B200_OK;
}

int fr_b200_decode_greedy(fr_b200_model *m, const int32_t *first_ids, int batch, int n_tokens, int32_t *out_ids,
                          void *stream) {
  if (!m || !first_ids || !out_ids) return fail(FR_B200_E_ARG, "null argument");
  if (!m->finalized) return fail(FR_B200_E_STATE, "finalize the model first");
  if (batch < 1 || batch > m->cfg.max_batch || n_tokens < 1) return fail(FR_B200_E_ARG, "bad batch or n_tokens");
  CU(cudaSetDevice(m->device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t need = (size_t)n_tokens * batch;
  if (m->hist_n < need) {
    CU(cudaStreamSynchronize(st));
    if (m->d_hist) cudaFree(m->d_hist);
    m->d_hist = nullptr; m->hist_n = 0;
    CU(cudaMalloc((void **)&m->d_hist, need * 12));
    m->hist_n = need;
  }
  if (decode_by_rows(m, batch)) {
    // GEMM path: ids stay on the device, row t of the history feeds step t + 1
    int rc = rows_decode_check(m, first_ids, batch, st);
    if (rc) return rc;
    int32_t *hist32 = reinterpret_cast<int32_t *>(m->d_hist + need);
    GreedyCtl ctl;
    ctl.hist = hist32; ctl.step = 0;
    CU(cudaMemcpyAsync(m->d_ctl, &ctl, sizeof(ctl), cudaMemcpyHostToDevice, st));
    // step 0 from the host ids; every sampled id goes to the row-id buffer of the next step and to the history
    if ((rc = rows_forward(m, true, 0, first_ids, batch, st))) return rc;
    int32_t *row_ids = reinterpret_cast<int32_t *>(m->d_seq);   // first piece of the activation blob
    CU(launch_argmax_rows(m->d_out, batch, m->V, m->Vpad, row_ids, m->d_ctl, st));
    m->launches += 2;
    int left = n_tokens - 1;
    bool graphs = left >= 4;
    if (const char *e = getenv("FR_B200_GRAPH")) graphs = graphs && atoi(e) != 0;
    if (graphs) {
      // two steps (the shift-state copies alternate) as one graph on an internal stream: capture is not allowed on the
      // legacy default stream, which is what most callers pass
      if (!m->gstream) {
        CU(cudaStreamCreateWithFlags(&m->gstream, cudaStreamNonBlocking));
        CU(cudaEventCreateWithFlags(&m->gev, cudaEventDisableTiming));
      }
      if (!m->gexec || m->g_batch != batch || m->g_par != m->par[0] || m->g_seq != m->d_seq) {
        if (m->gexec) { cudaGraphExecDestroy(m->gexec); m->gexec = nullptr; }
        const long long l0 = m->launches;
        cudaGraph_t graph = nullptr;
        bool ok = cudaStreamBeginCapture(m->gstream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        for (int i = 0; i < 2 && ok; ++i) {
          ok = rows_forward(m, true, 0, row_ids, batch, m->gstream) == 0 &&
               launch_argmax_rows(m->d_out, batch, m->V, m->Vpad, row_ids, m->d_ctl, m->gstream) == cudaSuccess;
        }
        cudaError_t ce = cudaStreamEndCapture(m->gstream, &graph);
        ok = ok && ce == cudaSuccess && graph && cudaGraphInstantiate(&m->gexec, graph, 0) == cudaSuccess;
        if (graph) cudaGraphDestroy(graph);
        m->launches = l0;
        if (!ok) {
          if (getenv("FR_B200_DEBUG")) fprintf(stderr, "fr_b200: graph capture failed (%s): running the steps one by one\n", cudaGetErrorString(ce));
          cudaGetLastError(); m->gexec = nullptr; graphs = false;
        }
        else { m->g_batch = batch; m->g_par = m->par[0]; m->g_seq = m->d_seq; }
      }
    }
    if (graphs && m->gexec) {
      const long long per_step = (m->v5 ? 9 : 7) * (long long)m->L + 4;
      CU(cudaEventRecord(m->gev, st));
      CU(cudaStreamWaitEvent(m->gstream, m->gev, 0));
      for (; left >= 2; left -= 2) {
        CU(cudaGraphLaunch(m->gexec, m->gstream));
        m->launches += 2 * per_step;
      }
      CU(cudaEventRecord(m->gev, m->gstream));
      CU(cudaStreamWaitEvent(st, m->gev, 0));
    }
    for (; left > 0; --left) {
      if ((rc = rows_forward(m, true, 0, row_ids, batch, st))) return rc;
      CU(launch_argmax_rows(m->d_out, batch, m->V, m->Vpad, row_ids, m->d_ctl, st));
      m->launches += 2;
    }
    CU(cudaMemcpyAsync(out_ids, hist32, need * 4, cudaMemcpyDefault, st));
    if (is_host_ptr(out_ids)) {
      int status = 0;
      CU(cudaMemcpyAsync(&status, m->out_status(), 4, cudaMemcpyDeviceToHost, st));
      CU(cudaStreamSynchronize(st));
      return check_status(m, status);
    }
    return FR_B200_OK;
  }
  // one packed arg-max word per (token, stream), all cleared up front; token t+1 reads its ids from row t
  CU(cudaMemsetAsync(m->d_hist, 0, need * 8, st));
  for (int t = 0; t < n_tokens; ++t) {
    int rc = decode_impl(m, t == 0 ? first_ids : nullptr, t == 0 ? nullptr : m->d_hist + (size_t)(t - 1) * batch, batch, st,
                         m->d_hist + (size_t)t * batch);
    if (rc) return rc;
  }
  int32_t *ids32 = reinterpret_cast<int32_t *>(m->d_hist + need);   // unpacked ids behind the packed words
  CU(launch_unpack_ids(m->d_hist, (int)need, ids32, st));
  m->launches++;
  if (is_host_ptr(out_ids)) {
    CU(cudaMemcpyAsync(out_ids, ids32, need * 4, cudaMemcpyDeviceToHost, st));
    int status = 0;
    CU(cudaMemcpyAsync(&status, m->out_status(), 4, cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    return check_status(m, status);
  }
  CU(cudaMemcpyAsync(out_ids, ids32, need * 4, cudaMemcpyDeviceToDevice, st));
  return FR_B200_OK;
}

int fr_b200_decode_profile(fr_b200_model *m, const int32_t *ids, int batch, uint64_t *stamps, int n_stamps) {
  if (!m || !ids || !stamps) return fail(FR_B200_E_ARG, "null argument");
  if (!m->finalized) return fail(FR_B200_E_STATE, "finalize the model first");
  if (batch < 1 || batch > m->cfg.max_batch) return fail(FR_B200_E_ARG, "batch must be 1..max_batch");
  if (decode_by_rows(m, batch)) return fail(FR_B200_E_UNSUPPORTED, "the trace exists for the persistent kernel (at most 8 streams) only");
  const int need = (int)m->phases.size() * 8 * m->grid;
  if (n_stamps < need) return fail(FR_B200_E_ARG, "stamps must hold 8 * n_phases * n_ctas entries");
  CU(cudaSetDevice(m->device));
  DevBuf buf;
  CU(buf.alloc((size_t)need * 8));
  CU(cudaMemset(buf.p, 0, (size_t)need * 8));
  int rc = decode_impl(m, ids, nullptr, batch, 0, nullptr, (unsigned long long *)buf.p);
  if (rc) return rc;
  CU(cudaDeviceSynchronize());
  CU(cudaMemcpy(stamps, buf.p, (size_t)need * 8, cudaMemcpyDeviceToHost));
  int status = 0;
  CU(cudaMemcpy(&status, m->out_status(), 4, cudaMemcpyDeviceToHost));
  return check_status(m, status);
}

int fr_b200_sample(fr_b200_model *m, int batch, float temperature, int top_k, float top_p, const float *uniform,
                   int32_t *ids, void *stream) {
  if (!m || !uniform || !ids) return fail(FR_B200_E_ARG, "null argument");
  if (!m->finalized) return fail(FR_B200_E_STATE, "finalize the model first");
  if (batch < 1 || batch > m->cfg.max_batch) return fail(FR_B200_E_ARG, "batch must be 1..max_batch");
  CU(cudaSetDevice(m->device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t need = sample_scratch_bytes(batch, m->V) + align256((size_t)batch * 4) * 2;
  if (m->sample_bytes < need) {
    CU(cudaStreamSynchronize(st));
    if (m->d_sample) cudaFree(m->d_sample);
    m->d_sample = nullptr; m->sample_bytes = 0;
    CU(cudaMalloc((void **)&m->d_sample, need));
    m->sample_bytes = need;
  }
  float *d_u = reinterpret_cast<float *>(m->d_sample);
  int32_t *d_ids = reinterpret_cast<int32_t *>(m->d_sample + align256((size_t)batch * 4));
  uint8_t *scratch = m->d_sample + 2 * align256((size_t)batch * 4);
  CU(cudaMemcpyAsync(d_u, uniform, (size_t)batch * 4, cudaMemcpyDefault, st));
  CU(launch_sample_rows(m->d_out, batch, m->V, m->Vpad, temperature, top_k, top_p, d_u, d_ids, scratch,
                        need - 2 * align256((size_t)batch * 4), st));
  m->launches += 4;
  CU(cudaMemcpyAsync(ids, d_ids, (size_t)batch * 4, cudaMemcpyDefault, st));
  if (is_host_ptr(ids)) CU(cudaStreamSynchronize(st));
  return FR_B200_OK;
}

int fr_b200_logits_add(fr_b200_model *m, int n, const int32_t *streams, const int32_t *tokens, const float *deltas, void *stream) {
  if (!m || n < 0 || (n > 0 && (!streams || !tokens || !deltas))) return fail(FR_B200_E_ARG, "bad argument");
  if (!m->finalized) return fail(FR_B200_E_STATE, "finalize the model first");
  if (n == 0) return FR_B200_OK;
  for (int i = 0; i < n; ++i)
    if (streams[i] < 0 || streams[i] >= m->cfg.max_batch || tokens[i] < 0 || tokens[i] >= m->V)
      return fail(FR_B200_E_ARG, "stream or token id out of range");
  CU(cudaSetDevice(m->device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t piece = align256((size_t)n * 4);
  if (m->adj_bytes < 3 * piece) {
    CU(cudaStreamSynchronize(st));
    if (m->d_adj) cudaFree(m->d_adj);
    m->d_adj = nullptr; m->adj_bytes = 0;
    CU(cudaMalloc((void **)&m->d_adj, 3 * piece));
    m->adj_bytes = 3 * piece;
  }
  CU(cudaMemcpyAsync(m->d_adj, streams, (size_t)n * 4, cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(m->d_adj + piece, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, st));
  CU(cudaMemcpyAsync(m->d_adj + 2 * piece, deltas, (size_t)n * 4, cudaMemcpyHostToDevice, st));
  CU(launch_logits_add(m->d_out, m->Vpad, reinterpret_cast<const int32_t *>(m->d_adj), reinterpret_cast<const int32_t *>(m->d_adj + piece),
                       reinterpret_cast<const float *>(m->d_adj + 2 * piece), n, st));
  CU(cudaStreamSynchronize(st));   // the host arrays were pageable: they may be reused once this returns
  m->launches++;
  return FR_B200_OK;
}

int fr_b200_logits_device(fr_b200_model *m, float **ptr) {
  if (!m || !ptr) return fail(FR_B200_E_ARG, "null argument");
  *ptr = m->d_out;
  return FR_B200_OK;
}
int fr_b200_vocab_padded(const fr_b200_model *m) { return m ? m->Vpad : FR_B200_E_ARG; }

namespace {

// The forward pass over R rows through [R, K] x [K, N] tensor-core GEMMs and row kernels.
//   seq mode   (batch_mode = false): the rows are the tokens of one prompt of stream `slot`
//              (def::ModelForwardSeq, kernels/default/model_forward_seq.cpp:48-184); logits of the last row only.
//   batch mode (batch_mode = true):  row b is the next token of stream b, b < R (the batched decode the reference
//              lacks); logits of every row into d_out.
// ids: host or device.  The residual stream stays fp32 between the layers; GEMM inputs are fp16.
int rows_forward(fr_b200_model *m, bool batch_mode, int slot, const int32_t *ids, int R, cudaStream_t st) {
  const int C = m->C, F = m->F, H = m->H, af = m->cfg.act_fp16, T = R;
  if (C > 8192) return fail(FR_B200_E_UNSUPPORTED, "the row kernels of the GEMM path hold at most n_embd = 8192");
  const size_t TC = (size_t)T * C, TF = (size_t)T * F;
  // activation buffers: one blob, 256-byte aligned pieces
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += align256(bytes); return o; };
  const size_t o_ids = take((size_t)T * 4), o_x = take(TC * 4), o_r = take(TC * 4), o_k = take(TC * 4), o_v = take(TC * 4),
               o_y = take(TC * 4), o_op0 = take(TC * 2), o_op1 = take(TC * 2), o_op2 = take(TC * 2), o_op3 = take(TC * 2),
               o_g = take(TC * 2), o_yn = take(TC * 2), o_kk = take(TF * 2), o_lo0 = take(TC * 2), o_lo1 = take(TC * 2),
               o_lo2 = take(batch_mode ? TC * 2 : 0), o_lo3 = take(batch_mode ? TC * 2 : 0), o_ynlo = take(batch_mode ? TC * 2 : 0),
               o_kklo = take(batch_mode ? TF * 2 : 0), o_glo = take(batch_mode ? TC * 2 : 0),
               o_raw = take(T <= GEMM_SMALL_M ? (size_t)GEMM_SPLIT_MAX * T * std::max(4 * C, F + C) * 4 : 0);   // split-K slabs
  // Long prompts are cut into pieces of rows that run on streams of their own, a layer apart: piece p's layer l needs
  // piece p's layer l - 1 (its stream order) and the recurrent state piece p - 1 left after layer l (an event), nothing
  // else -- the token shift crosses the cut through the stored shift state, like two prompts fed one after the other.
  // The tail wave of one piece's GEMM, its state scan and its row kernels then overlap the other piece's GEMMs.
  // (Not with host-visible state: kernels of two streams working on managed memory cost more than the overlap gains,
  // measured 11.6 against 7.8 ms for 4 layers of the 3B shape.)
  int n_pieces = 1;
  if (!batch_mode && T >= 2048 && !m->cfg.host_visible_state) {
    n_pieces = 2;
    if (const char *e = getenv("FR_B200_SEQ_PIECES")) n_pieces = std::max(1, std::min(atoi(e), 4));
    n_pieces = std::min(n_pieces, T / 512);
  }
  const int piece_rows = ((T + n_pieces - 1) / n_pieces + 255) / 256 * 256;   // whole 256-row GEMM tiles per piece
  n_pieces = (T + piece_rows - 1) / piece_rows;
  // state scan (seq mode, RWKV-5): enough chunks to cover the SMs a few times over, none shorter than 32 tokens
  const int Tp = std::min(T, piece_rows);
  int max_chunks = 1;
  if (!batch_mode && m->v5) max_chunks = std::max(1, std::min(Tp / 32, std::max(1, wkv5_scan_slots() / H)));
  const size_t scan_bytes = max_chunks > 1 ? (size_t)H * max_chunks * 4096 * 4 : 0;
  const size_t o_e = take(scan_bytes * n_pieces), o_sin = take(scan_bytes * n_pieces);
  if (m->seq_bytes < off) {
    CU(cudaStreamSynchronize(st));
    if (m->d_seq) cudaFree(m->d_seq);
    m->d_seq = nullptr; m->seq_bytes = 0;
    CU(cudaMalloc((void **)&m->d_seq, off));
    m->seq_bytes = off;
  }
  uint8_t *B = m->d_seq;
  int32_t *d_ids = (int32_t *)(B + o_ids);
  float *x = (float *)(B + o_x), *r_all = (float *)(B + o_r), *k_all = (float *)(B + o_k), *v_all = (float *)(B + o_v), *y_all = (float *)(B + o_y);
  __half *op_all[4] = {(__half *)(B + o_op0), (__half *)(B + o_op1), (__half *)(B + o_op2), (__half *)(B + o_op3)};
  __half *g_all = (__half *)(B + o_g), *yn_all = (__half *)(B + o_yn), *kk_all = (__half *)(B + o_kk);   // (the ffn receptance reuses g)
  __half *lo0_all = (__half *)(B + o_lo0), *lo1_all = (__half *)(B + o_lo1);
  // batch mode keeps every GEMM input as a hi + lo pair: the steps are bound by weight bytes, not flops, and the
  // per-stream error must not depend on how many streams share the step
  __half *lo2_all = batch_mode ? (__half *)(B + o_lo2) : nullptr, *lo3_all = batch_mode ? (__half *)(B + o_lo3) : nullptr;
  __half *ynlo_all = batch_mode ? (__half *)(B + o_ynlo) : nullptr, *kklo_all = batch_mode ? (__half *)(B + o_kklo) : nullptr;
  __half *glo_all = batch_mode ? (__half *)(B + o_glo) : nullptr;
  cudaStream_t st_main = st;
  if (ids != d_ids) CU(cudaMemcpyAsync(d_ids, ids, (size_t)T * 4, cudaMemcpyDefault, st));
  CU(launch_gather_emb(m->d_emb, m->emb_dtype == FR_B200_T_F32, d_ids, T, C, x, st));
  auto vp = [&](const std::string &n) -> const float * { return m->d_vecs + m->vecs[n].off; };
  const bool quant = m->fmt != FMT_FP16;
  auto mk = [&](int rows, const __half *A, const std::string &w, int N, int K, int epi, void *out, const void *aux0, const void *aux1,
                float scale, const __half *A2 = nullptr) -> GemmArgs {
    GemmArgs ga;
    memset(&ga, 0, sizeof(ga));
    const MatrixSlot &ms = m->mats[w];
    ga.A = A; ga.A2 = A2; ga.M = rows;
    if (quant) {
      ga.Wq = m->d_qcopy + ms.q_off; ga.wfmt = m->fmt;
      if (m->fmt == FMT_INT4) ga.wq_scale = m->d_qscale + ms.qs_off;
      else ga.col_scale = m->d_pscale + ms.pscale_off;
    } else {
      ga.Bt = m->d_plain + ms.plain_off;
    }
    ga.N = N; ga.K = K; ga.epi = epi; ga.out = out; ga.ldo = N; ga.aux0 = aux0; ga.aux1 = aux1;
    ga.scale = scale; ga.status = m->out_status();
    return ga;
  };
  const int mt = Tp > 128 ? 2 : 1;   // 256-row tiles once the rows fill them
  // few rows: every GEMM of a launch gets its own run of split-K slabs
  auto give_raw = [&](GemmArgs *grp, int n) {
    if (T > GEMM_SMALL_M) return;
    float *p = (float *)(B + o_raw);
    for (int i = 0; i < n; ++i) { grp[i].raw = p; p += (size_t)GEMM_SPLIT_MAX * T * grp[i].N; }
  };
  const int par0 = (int)m->par[batch_mode ? 0 : slot];
  const int nvec = m->v5 ? (m->gate ? 4 : 3) : 3;
  uint8_t *st0 = m->d_state + (batch_mode ? 0 : (size_t)slot * m->state_stride);
  // streams and events of the pieces (one piece: everything on the caller's stream)
  if (n_pieces > 1) {
    for (int pc = 0; pc < n_pieces; ++pc)
      if (!m->seq_streams[pc]) CU(cudaStreamCreateWithFlags(&m->seq_streams[pc], cudaStreamNonBlocking));
    while ((int)m->seq_events.size() < n_pieces * (m->L + 1)) {
      cudaEvent_t ev;
      CU(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
      m->seq_events.push_back(ev);
    }
    cudaEvent_t start = m->seq_events[n_pieces * m->L];          // everything before the layers (ids, embedding rows)
    CU(cudaEventRecord(start, st));
    for (int pc = 0; pc < n_pieces; ++pc) CU(cudaStreamWaitEvent(m->seq_streams[pc], start, 0));
  }
  float *const x_all = x;
  // Batch mode: a projection that was split over K leaves its slabs to the row kernel that follows it (the WKV step
  // after key / value / receptance, the LayerNorm after the two projections that add to x) instead of a finishing
  // pass of its own: three launches fewer per layer.
  struct Pending { const float *raw; const __half *cscale, *r, *r_lo; float scale; int split; } pend_x = {nullptr, nullptr, nullptr, nullptr, 1.f, 1};
  auto take_pending = [&](SeqLnArgs &la, float *xrows) {
    if (pend_x.split > 1) {
      la.pend_raw = pend_x.raw; la.pend_cscale = pend_x.cscale; la.pend_r = pend_x.r; la.pend_r_lo = pend_x.r_lo;
      la.pend_scale = pend_x.scale; la.pend_split = pend_x.split; la.x_wr = xrows;
    }
    pend_x.split = 1;
  };
  for (int l = 0; l < m->L; ++l)
  for (int pc = 0; pc < n_pieces; ++pc) {
    const std::string b = "blocks." + std::to_string(l) + ".", a = b + "att.", f = b + "ffn.";
    uint8_t *stb = st0 + (size_t)l * m->layer_stride;
    // this piece's rows of every activation buffer, its stream, its copy of the shift states (they alternate piece by
    // piece exactly as they alternate token by token) and its scan scratch
    const int t0 = pc * piece_rows, T = std::min(R, t0 + piece_rows) - t0;
    const size_t rc = (size_t)t0 * C, rf = (size_t)t0 * F;
    cudaStream_t st = n_pieces > 1 ? m->seq_streams[pc] : st_main;
    const int par = par0 ^ (pc & 1);
    float *x = x_all + rc, *r = r_all + rc, *k = k_all + rc, *v = v_all + rc, *y = y_all + rc;
    __half *op[4] = {op_all[0] + rc, op_all[1] + rc, op_all[2] + rc, op_all[3] + rc};
    __half *g = g_all + rc, *yn = yn_all + rc, *kk = kk_all + rf, *rr = g;
    __half *lo0 = lo0_all + rc, *lo1 = lo1_all + rc;
    __half *lo2 = lo2_all ? lo2_all + rc : nullptr, *lo3 = lo3_all ? lo3_all + rc : nullptr;
    __half *yn_lo = ynlo_all ? ynlo_all + rc : nullptr, *kk_lo = kklo_all ? kklo_all + rf : nullptr;
    __half *g_lo = glo_all ? glo_all + rc : nullptr, *rr_lo = g_lo;
    int n_chunks = 1, chunk_len = T;
    if (!batch_mode && m->v5) {
      n_chunks = std::max(1, std::min(T / 32, std::max(1, wkv5_scan_slots() / (H * n_pieces))));   // the pieces run side by side
      chunk_len = (T + n_chunks - 1) / n_chunks;
      n_chunks = (T + chunk_len - 1) / chunk_len;
    }
    if (n_pieces > 1 && pc > 0) CU(cudaStreamWaitEvent(st, m->seq_events[(pc - 1) * m->L + l], 0));   // the state after layer l of the rows before
    // ---- time mix ----
    SeqLnArgs la;
    memset(&la, 0, sizeof(la));
    la.x = x; la.ln_w = vp(b + "ln1.weight"); la.ln_b = vp(b + "ln1.bias");
    la.mix[0] = vp(a + "time_mix_k"); la.mix[1] = vp(a + "time_mix_v"); la.mix[2] = vp(a + "time_mix_r");
    if (m->gate) la.mix[3] = vp(a + "time_mix_g");
    for (int i = 0; i < 4; ++i) la.op[i] = op[i];
    la.sx_rd = stb + off_sx(C, af, par); la.sx_wr = stb + off_sx(C, af, par ^ 1);
    la.T = T; la.C = C; la.nvec = nvec; la.act_fp16 = af;
    la.batch_mode = batch_mode; la.state_stride = m->state_stride;
    // k and v build the recurrent state, which keeps growing with the prompt: their projections take the
    // activations as hi + lo fp16 pairs (a second pass over K), like every decode matvec does
    la.op_lo[0] = lo0; la.op_lo[1] = lo1; la.op_lo[2] = lo2; la.op_lo[3] = lo3;
    take_pending(la, x);
    CU(launch_ln_mix_seq(la, st));
    int kvr_split = 1;
    const __half *kvr_cs[3] = {nullptr, nullptr, nullptr};
    const float *kvr_raw[3] = {nullptr, nullptr, nullptr};
    {
      // the attention projections in one launch; the two with a second pass over K first
      GemmArgs grp[4] = {mk(T, op[0], a + "key.weight", C, C, GEMM_EPI_F32, k, nullptr, nullptr, 1.f, lo0),
                         mk(T, op[1], a + "value.weight", C, C, GEMM_EPI_F32, v, nullptr, nullptr, 1.f, lo1),
                         mk(T, op[2], a + "receptance.weight", C, C, GEMM_EPI_F32, r, nullptr, nullptr, 1.f, lo2),
                         mk(T, op[2], a + "receptance.weight", C, C, GEMM_EPI_F32, r, nullptr, nullptr, 1.f, lo2)};
      if (m->gate) { grp[3] = mk(T, op[3], a + "gate.weight", C, C, GEMM_EPI_SILU_F16, g, nullptr, nullptr, 1.f, lo3); grp[3].out_lo = g_lo; }
      give_raw(grp, m->gate ? 4 : 3);
      const bool defer = batch_mode && !m->v5;
      CU(launch_gemm_group(grp, m->gate ? 4 : 3, mt, st, defer ? &kvr_split : nullptr));
      for (int i = 0; i < 3; ++i) { kvr_cs[i] = grp[i].col_scale; kvr_raw[i] = grp[i].raw; }
    }
    if (m->v5) {
      SeqWkvArgs wa;
      memset(&wa, 0, sizeof(wa));
      wa.r = r; wa.k = k; wa.v = v; wa.decay = vp(a + "time_decay"); wa.first = vp(a + "time_first");
      wa.state = reinterpret_cast<float *>(stb + off_mid(C, af)); wa.y = y; wa.T = T; wa.C = C;
      wa.per_head = m->cfg.version == FR_B200_V5_0;
      wa.n_chunks = n_chunks; wa.chunk_len = chunk_len; wa.e_out = (float *)(B + o_e + scan_bytes * pc); wa.s_in = (float *)(B + o_sin + scan_bytes * pc);
      wa.batch_mode = batch_mode; wa.state_stride = m->state_stride / 4;
      CU(launch_wkv5_seq(wa, H, st));
      CU(launch_gn_gate_seq(y, vp(a + "ln_x.weight"), vp(a + "ln_x.bias"), m->gate ? g : nullptr, m->gate ? g_lo : nullptr, T, H, yn, yn_lo, st));
    } else {
      Wkv4Args wa;
      memset(&wa, 0, sizeof(wa));
      wa.k = k; wa.v = v; wa.r = r; wa.decay = vp(a + "time_decay"); wa.first = vp(a + "time_first");
      wa.state = stb + off_mid(C, af); wa.state_stride = m->state_stride; wa.out = yn; wa.out_lo = yn_lo; wa.T = T; wa.C = C; wa.batch_mode = batch_mode;
      if (kvr_split > 1) {
        wa.split = kvr_split;
        wa.raw_k = kvr_raw[0]; wa.raw_v = kvr_raw[1]; wa.raw_r = kvr_raw[2];
        wa.cs_k = kvr_cs[0]; wa.cs_v = kvr_cs[1]; wa.cs_r = kvr_cs[2];
      }
      CU(launch_wkv4_rows(wa, st));
    }
    {
      GemmArgs go = mk(T, yn, a + "output.weight", C, C, GEMM_EPI_ADD_F32, x, x, nullptr, 1.f, yn_lo);
      give_raw(&go, 1);
      // prompts: few tiles, 128-row tiles fill the SMs better (measured); streams: one pass over the weights for all rows
      int sp = 1;
      CU(launch_gemm_group(&go, 1, batch_mode ? mt : 1, st, batch_mode ? &sp : nullptr));
      if (sp > 1) pend_x = {go.raw, go.col_scale, nullptr, nullptr, go.scale, sp};
    }
    // ---- channel mix ----
    memset(&la, 0, sizeof(la));
    la.x = x; la.ln_w = vp(b + "ln2.weight"); la.ln_b = vp(b + "ln2.bias");
    la.mix[0] = vp(f + "time_mix_k"); la.mix[1] = vp(f + "time_mix_r");
    la.op[0] = op[0]; la.op[1] = op[1];
    la.op_lo[0] = batch_mode ? lo0 : nullptr; la.op_lo[1] = batch_mode ? lo1 : nullptr;
    la.sx_rd = stb + off_ffn_sx(C, H, m->v5, af, par); la.sx_wr = stb + off_ffn_sx(C, H, m->v5, af, par ^ 1);
    la.T = T; la.C = C; la.nvec = 2; la.act_fp16 = af;
    la.batch_mode = batch_mode; la.state_stride = m->state_stride;
    take_pending(la, x);
    CU(launch_ln_mix_seq(la, st));
    const bool halve = af && (l + 1) % 6 == 0;   // x / 2 every 6 layers under fp16 activations (model_forward_seq.cpp:165-167)
    {
      GemmArgs grp[2] = {mk(T, op[0], f + "key.weight", F, C, GEMM_EPI_RELU2_F16, kk, nullptr, nullptr, 1.f, batch_mode ? lo0 : nullptr),
                         mk(T, op[1], f + "receptance.weight", C, C, GEMM_EPI_SIGMOID_F16, rr, nullptr, nullptr, 1.f, batch_mode ? lo1 : nullptr)};
      grp[0].out_lo = kk_lo; grp[1].out_lo = rr_lo;
      give_raw(grp, 2);
      CU(launch_gemm_group(grp, 2, mt, st));
      GemmArgs gv = mk(T, kk, f + "value.weight", C, F, GEMM_EPI_MULADD_F32, x, x, rr, halve ? 0.5f : 1.f, kk_lo);
      gv.aux1_lo = rr_lo;
      give_raw(&gv, 1);
      int sp = 1;
      CU(launch_gemm_group(&gv, 1, batch_mode ? mt : 1, st, batch_mode ? &sp : nullptr));
      if (sp > 1) pend_x = {gv.raw, gv.col_scale, rr, rr_lo, gv.scale, sp};
    }
    m->launches += m->v5 ? 9 : 7;
    if (n_pieces > 1) CU(cudaEventRecord(m->seq_events[pc * m->L + l], st));
  }
  if (n_pieces > 1) {
    // back on the caller's stream once every piece has finished its last layer
    for (int pc = 0; pc < n_pieces; ++pc) CU(cudaStreamWaitEvent(st_main, m->seq_events[pc * m->L + m->L - 1], 0));
  }
  if (batch_mode) {
    // every row: ln_out, then the head as one more GEMM -> fp32 logits [R, Vpad]
    SeqLnArgs la;
    memset(&la, 0, sizeof(la));
    la.x = x; la.ln_w = vp("ln_out.weight"); la.ln_b = vp("ln_out.bias"); la.op[0] = op_all[0]; la.op_lo[0] = lo0_all;
    la.T = T; la.C = C; la.nvec = 0; la.act_fp16 = af; la.batch_mode = 1;
    take_pending(la, x);
    CU(launch_ln_mix_seq(la, st));
    GemmArgs gh = mk(T, op_all[0], "head.weight", m->V, C, GEMM_EPI_F32, m->d_out, nullptr, nullptr, 1.f, lo0_all);
    gh.ldo = m->Vpad;
    // (no split-K scratch for the head: it has a thousand column tiles of its own)
    CU(launch_gemm_group(&gh, 1, mt, st));
    m->launches += 2;
    for (int bq = 0; bq < R; ++bq) m->par[bq] ^= 1u;
    return 0;
  }
  // last token -> ln_out -> head, as a stand-alone matvec over the head's streaming tiles
  CU(launch_ln_row(x + (size_t)(T - 1) * C, vp("ln_out.weight"), vp("ln_out.bias"), C, m->d_lnvec, st));
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.version = 4; p.L = 0; p.C = 64; p.F = C; p.V = m->V; p.Vpad = m->Vpad; p.fmt = m->fmt; p.B = 1; p.n_phases = 1;
  p.phases = m->d_head_phase; p.kk = reinterpret_cast<exch_t *>(m->d_lnvec);   // PH_MATVEC reads kk as plain fp32
  p.logits = m->d_out + (size_t)slot * m->Vpad; p.status = m->out_status();
  int optin = 0, stages = 0;
  CU(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, m->device));
  for (int sg = 6; sg >= 2; --sg)
    if (decode_smem_bytes(m->fmt, 0, 64, C, 4, sg) <= (size_t)optin) { stages = sg; break; }
  if (!stages) return fail(FR_B200_E_UNSUPPORTED, "n_embd too large for the head matvec");
  p.n_stages = stages;
  const size_t smem = decode_smem_bytes(m->fmt, 0, 64, C, 4, stages);
  int grid = 0;
  CU(decode_max_grid(m->fmt, 0, smem, m->device, &grid));
  if (!grid) return fail(FR_B200_E_UNSUPPORTED, "kernel does not fit");
  CU(launch_decode(p, 0, grid, smem, st));
  m->launches += 3;
  if (n_pieces & 1) m->par[slot] ^= 1u;   // every piece flipped the shift-state copies once
  return 0;
}

}  // namespace

int fr_b200_run_seq(fr_b200_model *m, int slot, const int32_t *ids, int n, float *last_logits, void *stream) {
  if (!m || !ids || n < 1) return fail(FR_B200_E_ARG, "bad argument");
  if (!m->finalized) return fail(FR_B200_E_STATE, "finalize the model first");
  if (slot < 0 || slot >= m->cfg.max_batch) return fail(FR_B200_E_ARG, "slot out of range");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int seq_min = 2;   // shorter prompts take the token loop
  if (const char *e = getenv("FR_B200_SEQ_MIN")) seq_min = atoi(e);
  // fp16 RWKV-4 models build their row copies when the first prompt of 32 tokens or more arrives
  bool by_rows = rows_path_built(m) && n >= seq_min;
  if (!by_rows && m->fmt == FMT_FP16 && m->row_copies && m->plain_halfs && n >= std::max(seq_min, 32)) {
    CU(cudaSetDevice(m->device));
    int rc = ensure_row_copies(m);
    if (rc) return rc;
    by_rows = true;
  }
  if (by_rows) {
    CU(cudaSetDevice(m->device));
    for (int i = 0; i < n; ++i)
      if (ids[i] < 0 || ids[i] >= m->V) return fail(FR_B200_E_ARG, "token id out of range");
    int rc = rows_forward(m, false, slot, ids, n, st);
    if (rc) return rc;
    if (last_logits) {
      if (is_host_ptr(last_logits)) {
        CU(cudaMemcpyAsync(m->h_out, m->d_out + (size_t)slot * m->Vpad, (size_t)m->V * 4, cudaMemcpyDeviceToHost, st));
      } else {
        CU(cudaMemcpyAsync(last_logits, m->d_out + (size_t)slot * m->Vpad, (size_t)m->V * 4, cudaMemcpyDeviceToDevice, st));
      }
    }
    CU(cudaStreamSynchronize(st));
    int status = 0;
    CU(cudaMemcpy(&status, m->out_status(), 4, cudaMemcpyDeviceToHost));
    if ((rc = check_status(m, status))) return rc;
    if (last_logits && is_host_ptr(last_logits)) memcpy(last_logits, m->h_out, (size_t)m->V * 4);
    return FR_B200_OK;
  }
  if (slot != 0) return fail(FR_B200_E_UNSUPPORTED, "the token loop of run_seq uses stream slot 0");
  for (int i = 0; i < n; ++i) {
    int rc = fr_b200_decode(m, ids + i, 1, i == n - 1 ? last_logits : nullptr, nullptr, stream);
    if (rc) return rc;
  }
  if (!last_logits) {
    CU(cudaStreamSynchronize(st));
    int status = 0;
    CU(cudaMemcpy(&status, m->out_status(), 4, cudaMemcpyDeviceToHost));
    return check_status(m, status);
  }
  return FR_B200_OK;
}

// ---- state ---------------------------------------------------------------------------------------

int fr_b200_state_count(const fr_b200_model *m) { return m ? (m->v5 ? 3 : 5) : FR_B200_E_ARG; }

int fr_b200_state_tensor(fr_b200_model *m, int slot, int layer, int index, void **dev_ptr, int *dtype, int64_t *numel) {
  if (!m) return fail(FR_B200_E_ARG, "null model");
  if (slot < 0 || slot >= m->cfg.max_batch || layer < 0 || layer >= m->L || index < 0 || index >= fr_b200_state_count(m))
    return fail(FR_B200_E_ARG, "state index out of range");
  const int af = m->cfg.act_fp16, C = m->C, par = (int)m->par[slot];
  uint8_t *base = m->d_state + (size_t)slot * m->state_stride + (size_t)layer * m->layer_stride;
  size_t off = 0; int64_t n = C; int dt = af ? FR_B200_T_F16 : FR_B200_T_F32;
  const int last = m->v5 ? 2 : 4;
  if (index == 0) off = off_sx(C, af, par);
  else if (index == last) off = off_ffn_sx(C, m->H, m->v5, af, par);
  else if (m->v5) { off = off_mid(C, af); n = (int64_t)m->H * 4096; dt = FR_B200_T_F32; }
  else { off = off_mid(C, af) + (size_t)(index - 1) * C * 4; dt = FR_B200_T_F32; }
  if (dev_ptr) *dev_ptr = base + off;
  if (dtype) *dtype = dt;
  if (numel) *numel = n;
  return FR_B200_OK;
}

// logical state of one slot = the reference's tensors back to back (sx, aa, bb, pp, ffn_sx per layer, or
// sx, s, ffn_sx), taken from / written to the copy of the token-shift states the next token will read
static int state_copy(fr_b200_model *m, int slot, uint8_t *ext, bool to_ext) {
  const int cnt = fr_b200_state_count(m);
  size_t pos = 0;
  for (int l = 0; l < m->L; ++l)
    for (int i = 0; i < cnt; ++i) {
      void *ptr; int dt; int64_t n;
      int rc = fr_b200_state_tensor(m, slot, l, i, &ptr, &dt, &n);
      if (rc) return rc;
      const size_t bytes = (size_t)n * (dt == FR_B200_T_F16 ? 2 : 4);
      if (to_ext) CU(cudaMemcpy(ext + pos, ptr, bytes, cudaMemcpyDefault));
      else CU(cudaMemcpy(ptr, ext + pos, bytes, cudaMemcpyDefault));
      pos += bytes;
    }
  return FR_B200_OK;
}

size_t fr_b200_state_bytes(const fr_b200_model *m) {
  if (!m) return 0;
  return (size_t)m->L * (2 * (size_t)m->C * act_bytes(m->cfg.act_fp16) + mid_bytes(m->C, m->H, m->v5));
}

int fr_b200_state_reset(fr_b200_model *m, int slot) {
  if (!m) return fail(FR_B200_E_ARG, "null model");
  if (slot < -1 || slot >= m->cfg.max_batch) return fail(FR_B200_E_ARG, "slot out of range");
  CU(cudaSetDevice(m->device));
  const size_t per = m->layer_stride * m->L;
  std::vector<uint8_t> h(per, 0);
  if (!m->v5) {
    // pp = -1e30 (model.cpp:157-158)
    for (int l = 0; l < m->L; ++l) {
      float *pp = reinterpret_cast<float *>(h.data() + (size_t)l * m->layer_stride + off_mid(m->C, m->cfg.act_fp16) + 2 * (size_t)m->C * 4);
      for (int i = 0; i < m->C; ++i) pp[i] = -1e30f;
    }
  }
  for (int s = 0; s < m->cfg.max_batch; ++s)
    if (slot < 0 || slot == s) {
      CU(cudaMemcpy(m->d_state + (size_t)s * m->state_stride, h.data(), per, cudaMemcpyHostToDevice));
      m->par[s] = 0;
    }
  return FR_B200_OK;
}

int fr_b200_state_export(fr_b200_model *m, int slot, void *dst, size_t dst_bytes) {
  if (!m || !dst) return fail(FR_B200_E_ARG, "null argument");
  if (slot < 0 || slot >= m->cfg.max_batch) return fail(FR_B200_E_ARG, "slot out of range");
  if (dst_bytes < fr_b200_state_bytes(m)) return fail(FR_B200_E_ARG, "destination too small");
  CU(cudaSetDevice(m->device));
  CU(cudaDeviceSynchronize());
  return state_copy(m, slot, static_cast<uint8_t *>(dst), true);
}

int fr_b200_state_import(fr_b200_model *m, int slot, const void *src, size_t src_bytes) {
  if (!m || !src) return fail(FR_B200_E_ARG, "null argument");
  if (slot < 0 || slot >= m->cfg.max_batch) return fail(FR_B200_E_ARG, "slot out of range");
  if (src_bytes != fr_b200_state_bytes(m)) return fail(FR_B200_E_ARG, "state size mismatch");
  CU(cudaSetDevice(m->device));
  CU(cudaDeviceSynchronize());
  return state_copy(m, slot, const_cast<uint8_t *>(static_cast<const uint8_t *>(src)), false);
}

// ---- quantisers -----------------------------------------------------------------------------------

int fr_b200_quantize_int8(const float *W, int K, int N, int8_t *q, uint16_t *scales, int device) {
  if (!W || !q || !scales || K <= 0 || N <= 0) return fail(FR_B200_E_ARG, "bad argument");
  CU(cudaSetDevice(device));
  DevBuf dw, dq, ds;
  CU(dw.alloc((size_t)K * N * 4)); CU(dq.alloc((size_t)K * N)); CU(ds.alloc((size_t)N * 2));
  CU(cudaMemcpy(dw.p, W, (size_t)K * N * 4, cudaMemcpyDefault));
  CU(launch_quant_int8((const float *)dw.p, K, N, (int8_t *)dq.p, (__half *)ds.p, 0));
  CU(cudaMemcpy(q, dq.p, (size_t)K * N, cudaMemcpyDefault));
  CU(cudaMemcpy(scales, ds.p, (size_t)N * 2, cudaMemcpyDefault));
  return FR_B200_OK;
}
int fr_b200_quantize_int4(const float *W, int K, int N, uint8_t *packed, uint16_t *scales, int device) {
  if (!W || !packed || !scales || K <= 0 || N <= 0 || K % 32) return fail(FR_B200_E_ARG, "bad argument (K must be a multiple of 32)");
  CU(cudaSetDevice(device));
  DevBuf dw, dq, ds;
  CU(dw.alloc((size_t)K * N * 4)); CU(dq.alloc((size_t)K * N / 2)); CU(ds.alloc((size_t)N * (K / 32) * 2));
  CU(cudaMemcpy(dw.p, W, (size_t)K * N * 4, cudaMemcpyDefault));
  CU(launch_quant_int4((const float *)dw.p, K, N, (uint8_t *)dq.p, (__half *)ds.p, 0));
  CU(cudaMemcpy(packed, dq.p, (size_t)K * N / 2, cudaMemcpyDefault));
  CU(cudaMemcpy(scales, ds.p, (size_t)N * (K / 32) * 2, cudaMemcpyDefault));
  return FR_B200_OK;
}
int fr_b200_dequantize_int8(const int8_t *q, const uint16_t *scales, int K, int N, float *W, int device) {
  if (!W || !q || !scales || K <= 0 || N <= 0) return fail(FR_B200_E_ARG, "bad argument");
  CU(cudaSetDevice(device));
  DevBuf dw, dq, ds;
  CU(dw.alloc((size_t)K * N * 4)); CU(dq.alloc((size_t)K * N)); CU(ds.alloc((size_t)N * 2));
  CU(cudaMemcpy(dq.p, q, (size_t)K * N, cudaMemcpyDefault));
  CU(cudaMemcpy(ds.p, scales, (size_t)N * 2, cudaMemcpyDefault));
  CU(launch_dequant_int8((const int8_t *)dq.p, (const __half *)ds.p, K, N, (float *)dw.p, 0));
  CU(cudaMemcpy(W, dw.p, (size_t)K * N * 4, cudaMemcpyDefault));
  return FR_B200_OK;
}
int fr_b200_dequantize_int4(const uint8_t *packed, const uint16_t *scales, int K, int N, float *W, int device) {
  if (!W || !packed || !scales || K <= 0 || N <= 0 || K % 32) return fail(FR_B200_E_ARG, "bad argument");
  CU(cudaSetDevice(device));
  DevBuf dw, dq, ds;
  CU(dw.alloc((size_t)K * N * 4)); CU(dq.alloc((size_t)K * N / 2)); CU(ds.alloc((size_t)N * (K / 32) * 2));
  CU(cudaMemcpy(dq.p, packed, (size_t)K * N / 2, cudaMemcpyDefault));
  CU(cudaMemcpy(ds.p, scales, (size_t)N * (K / 32) * 2, cudaMemcpyDefault));
  CU(launch_dequant_int4((const uint8_t *)dq.p, (const __half *)ds.p, K, N, (float *)dw.p, 0));
  CU(cudaMemcpy(W, dw.p, (size_t)K * N * 4, cudaMemcpyDefault));
  return FR_B200_OK;
}

int fr_b200_unpack_matrix(fr_b200_model *m, const char *name, float *W, int K, int N) {
  if (!m || !name || !W) return fail(FR_B200_E_ARG, "null argument");
  auto it = m->mats.find(name);
  if (it == m->mats.end()) return fail(FR_B200_E_ARG, std::string("unknown matrix ") + name);
  const MatrixSlot &s = it->second;
  if (!s.set) return fail(FR_B200_E_STATE, "matrix not uploaded yet");
  if (K != s.K || N != s.N) return fail(FR_B200_E_ARG, "shape mismatch");
  CU(cudaSetDevice(m->device));
  DevBuf dw;
  CU(dw.alloc((size_t)K * N * 4));
  CU(launch_unpack(m->fmt, m->d_weights + s.tile_off, s.item_stride, m->d_rscale + s.rscale_off, s.rscale_stride, K, N,
                   (float *)dw.p, 0));
  CU(cudaMemcpy(W, dw.p, (size_t)K * N * 4, cudaMemcpyDefault));
  return FR_B200_OK;
}

int fr_b200_gemm_f16(const float *A, const float *W, int M, int N, int K, int epilogue, const float *aux0,
                     const float *aux1, float scale, float *out, int device) {
  if (!A || !W || !out || M < 1 || N < 1 || K < 64 || K % 64) return fail(FR_B200_E_ARG, "bad argument (K must be a positive multiple of 64)");
  if (epilogue < 0 || epilogue > GEMM_EPI_PLAIN_F16) return fail(FR_B200_E_ARG, "bad epilogue");
  if ((epilogue == GEMM_EPI_ADD_F32 || epilogue == GEMM_EPI_MULADD_F32) && !aux0) return fail(FR_B200_E_ARG, "aux0 missing");
  if (epilogue == GEMM_EPI_MULADD_F32 && !aux1) return fail(FR_B200_E_ARG, "aux1 missing");
  CU(cudaSetDevice(device));
  const size_t na = (size_t)M * K, nw = (size_t)K * N, no = (size_t)M * N;
  DevBuf a32, a16, w32, w16, wt, o, x0, r32, r16, st;
  CU(a32.alloc(na * 4)); CU(a16.alloc(na * 2)); CU(w32.alloc(nw * 4)); CU(w16.alloc(nw * 2)); CU(wt.alloc(nw * 2));
  CU(o.alloc(no * 4)); CU(st.alloc(4));
  CU(cudaMemset(st.p, 0, 4));
  CU(cudaMemcpy(a32.p, A, na * 4, cudaMemcpyDefault));
  CU(cudaMemcpy(w32.p, W, nw * 4, cudaMemcpyDefault));
  CU(launch_f32_to_f16((const float *)a32.p, (__half *)a16.p, na, 0));
  CU(launch_f32_to_f16((const float *)w32.p, (__half *)w16.p, nw, 0));
  CU(launch_transpose_f16((const __half *)w16.p, K, N, (__half *)wt.p, 0));
  GemmArgs g;
  memset(&g, 0, sizeof(g));
  g.A = (const __half *)a16.p; g.Bt = (const __half *)wt.p; g.M = M; g.N = N; g.K = K; g.epi = epilogue;
  g.out = o.p; g.ldo = N; g.scale = scale; g.status = (int *)st.p;
  if (aux0) { CU(x0.alloc(no * 4)); CU(cudaMemcpy(x0.p, aux0, no * 4, cudaMemcpyDefault)); g.aux0 = x0.p; }
  if (aux1) {
    CU(r32.alloc(no * 4)); CU(r16.alloc(no * 2));
    CU(cudaMemcpy(r32.p, aux1, no * 4, cudaMemcpyDefault));
    CU(launch_f32_to_f16((const float *)r32.p, (__half *)r16.p, no, 0));
    g.aux1 = r16.p;
  }
  const bool half_out = epilogue == GEMM_EPI_SILU_F16 || epilogue == GEMM_EPI_SIGMOID_F16 || epilogue == GEMM_EPI_RELU2_F16 ||
                        epilogue == GEMM_EPI_PLAIN_F16;
  CU(launch_gemm_f16(g, 0));
  CU(cudaDeviceSynchronize());
  int status = 0;
  CU(cudaMemcpy(&status, st.p, 4, cudaMemcpyDeviceToHost));
  if (status) return fail(FR_B200_E_TIMEOUT, "device-side wait timed out (code " + std::to_string(status) + ")");
  if (half_out) {
    DevBuf o32;
    CU(o32.alloc(no * 4));
    CU(launch_f16_to_f32((const __half *)o.p, (float *)o32.p, no, 0));
    CU(cudaMemcpy(out, o32.p, no * 4, cudaMemcpyDefault));
  } else {
    CU(cudaMemcpy(out, o.p, no * 4, cudaMemcpyDefault));
  }
  return FR_B200_OK;
}

int fr_b200_matvec(const float *W, int K, int N, int weight_format, const float *x, int batch, float *y, int device) {
  if (!W || !x || !y || K <= 0 || N <= 0 || K % 64) return fail(FR_B200_E_ARG, "bad argument (K must be a positive multiple of 64)");
  if (weight_format < 0 || weight_format > 2) return fail(FR_B200_E_ARG, "bad weight_format");
  if (batch < 1 || batch > MAX_B) return fail(FR_B200_E_ARG, "batch must be 1..8");
  CU(cudaSetDevice(device));
  const int fmt = weight_format, Npad = (N + ROWS - 1) / ROWS * ROWS, nb = Npad / ROWS;
  const size_t rb = rowblock_bytes(fmt, K), n = (size_t)K * N;
  DevBuf dW, dW16, dq, ds, dt, drs, dx, dy, dph;
  CU(dW.alloc(n * 4)); CU(dt.alloc(rb * nb)); CU(drs.alloc((size_t)Npad * 2)); CU(dx.alloc((size_t)batch * K * 4));
  CU(dy.alloc(((size_t)batch * Npad + 1) * 4)); CU(dph.alloc(sizeof(PhaseDev)));
  CU(cudaMemcpy(dW.p, W, n * 4, cudaMemcpyDefault));
  CU(cudaMemcpy(dx.p, x, (size_t)batch * K * 4, cudaMemcpyDefault));
  CU(cudaMemset(dy.p, 0, ((size_t)batch * Npad + 1) * 4));
  CU(cudaMemset(drs.p, 0, (size_t)Npad * 2));
  if (fmt == FMT_FP16) {
    CU(dW16.alloc(n * 2));
    CU(launch_f32_to_f16((const float *)dW.p, (__half *)dW16.p, n, 0));
    CU(launch_pack(fmt, dW16.p, nullptr, K, N, (uint8_t *)dt.p, rb, nullptr, 0, 0));
  } else if (fmt == FMT_INT8) {
    CU(dq.alloc(n)); CU(ds.alloc((size_t)N * 2));
    CU(launch_quant_int8((const float *)dW.p, K, N, (int8_t *)dq.p, (__half *)ds.p, 0));
    CU(launch_pack(fmt, dq.p, (const __half *)ds.p, K, N, (uint8_t *)dt.p, rb, (__half *)drs.p, ROWS, 0));
  } else {
    CU(dq.alloc(n / 2)); CU(ds.alloc((size_t)N * (K / 32) * 2));
    CU(launch_quant_int4((const float *)dW.p, K, N, (uint8_t *)dq.p, (__half *)ds.p, 0));
    CU(launch_pack(fmt, dq.p, (const __half *)ds.p, K, N, (uint8_t *)dt.p, rb, nullptr, 0, 0));
  }
  PhaseDev ph;
  memset(&ph, 0, sizeof(ph));
  ph.w = (const uint8_t *)dt.p; ph.rscale = (const __half *)drs.p; ph.kind = PH_MATVEC; ph.K = K; ph.n_items = nb; ph.n_sub = 1;
  CU(cudaMemcpy(dph.p, &ph, sizeof(ph), cudaMemcpyHostToDevice));
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  // C only sizes the operand space, max(3*C, F) * batch halfs
  p.version = 4; p.L = 0; p.C = 64; p.F = K; p.V = N; p.Vpad = Npad; p.fmt = fmt; p.B = batch; p.n_phases = 1;
  p.phases = (const PhaseDev *)dph.p; p.kk = (exch_t *)dx.p; p.logits = (float *)dy.p;   // PH_MATVEC reads kk as plain fp32
  p.status = (int *)((float *)dy.p + (size_t)batch * Npad);
  const int mode = decode_mode(batch);
  int optin = 0, grid = 0;
  CU(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  int stages = 0;
  for (int s = 6; s >= 2; --s)
    if (decode_smem_bytes(fmt, mode, 64, K, 4, s) <= (size_t)optin) { stages = s; break; }
  if (!stages) return fail(FR_B200_E_UNSUPPORTED, "K too large for shared memory");
  p.n_stages = stages;
  const size_t smem = decode_smem_bytes(fmt, mode, 64, K, 4, stages);
  CU(decode_max_grid(fmt, mode, smem, device, &grid));
  if (!grid) return fail(FR_B200_E_UNSUPPORTED, "kernel does not fit");
  CU(launch_decode(p, mode, grid, smem, 0));
  CU(cudaDeviceSynchronize());
  int status = 0;
  CU(cudaMemcpy(&status, p.status, 4, cudaMemcpyDeviceToHost));
  if (status) return fail(FR_B200_E_TIMEOUT, "device-side wait timed out (code " + std::to_string(status) + ")");
  CU(cudaMemcpy2D(y, (size_t)N * 4, dy.p, (size_t)Npad * 4, (size_t)N * 4, batch, cudaMemcpyDefault));
  return FR_B200_OK;
}

int fr_b200_wait_selftest(int device, unsigned limit_us) {
  if (limit_us < 1 || limit_us > 1000000) return fail(FR_B200_E_ARG, "limit must be 1 .. 1,000,000 microseconds");
  CU(cudaSetDevice(device));
  DevBuf st;
  CU(st.alloc(4));
  CU(cudaMemset(st.p, 0, 4));
  CU(launch_wait_selftest((int *)st.p, (unsigned long long)limit_us * 1000ull, 0));
  CU(cudaDeviceSynchronize());
  int status = 0;
  CU(cudaMemcpy(&status, st.p, 4, cudaMemcpyDeviceToHost));
  if (status) return fail(FR_B200_E_TIMEOUT, "device-side wait timed out (code " + std::to_string(status) + ")");
  return FR_B200_OK;
}

// ---- packed model files ---------------------------------------------------------------------------------------------
// A finalized model's device blobs, written back to back behind a small header: the streaming tiles (quantised
// already), row scales, per-layer vectors, the embedding table and, for int8 / int4, the row-major packed copies.
// Loading one is a handful of large reads and host-to-device copies: no msgpack parse, no per-row embedding uploads,
// no re-quantisation (def::init_model, kernels/default/init_model.cpp:19-52,128-132, does all three on every start).
namespace {
struct PackedHeader {
  char magic[8];             // "FRB200P2"
  fr_b200_config cfg;        // max_batch / device / host_visible_state of the writer: replaced at load
  int32_t emb_dtype, has_row_copies;
  uint64_t weights_bytes, rscale_n, vecs_n, emb_bytes, qcopy_bytes, qscale_halfs, pscale_halfs;
};
constexpr size_t IO_CHUNK = 64u << 20;

int write_blob(FILE *f, const void *dev, size_t bytes, void *pinned) {
  for (size_t off = 0; off < bytes; off += IO_CHUNK) {
    const size_t n = std::min(IO_CHUNK, bytes - off);
    CU(cudaMemcpy(pinned, static_cast<const uint8_t *>(dev) + off, n, cudaMemcpyDeviceToHost));
    if (fwrite(pinned, 1, n, f) != n) return fail(FR_B200_E_ARG, "short write to the packed model file");
  }
  return 0;
}
int read_blob(FILE *f, void *dev, size_t bytes, void *pinned) {
  for (size_t off = 0; off < bytes; off += IO_CHUNK) {
    const size_t n = std::min(IO_CHUNK, bytes - off);
    if (fread(pinned, 1, n, f) != n) return fail(FR_B200_E_ARG, "packed model file is truncated");
    CU(cudaMemcpy(static_cast<uint8_t *>(dev) + off, pinned, n, cudaMemcpyHostToDevice));
  }
  return 0;
}
struct PinnedBuf {
  void *p = nullptr;
  ~PinnedBuf() { if (p) cudaFreeHost(p); }
};
}  // namespace

int fr_b200_save_packed(fr_b200_model *m, const char *path) {
  if (!m || !path) return fail(FR_B200_E_ARG, "null argument");
  if (!m->finalized) return fail(FR_B200_E_STATE, "finalize the model first");
  CU(cudaSetDevice(m->device));
  CU(cudaDeviceSynchronize());
  PackedHeader h;
  memset(&h, 0, sizeof(h));
  memcpy(h.magic, "FRB200P2", 8);
  h.cfg = m->cfg;
  h.emb_dtype = m->emb_dtype;
  h.has_row_copies = m->d_qcopy != nullptr;
  h.weights_bytes = m->weights_bytes; h.rscale_n = m->rscale_n; h.vecs_n = m->vecs_n;
  h.emb_bytes = (uint64_t)m->V * m->C * (m->emb_dtype == FR_B200_T_F16 ? 2 : 4);
  h.qcopy_bytes = m->d_qcopy ? m->qcopy_bytes : 0; h.qscale_halfs = m->d_qscale ? m->qscale_halfs : 0;
  h.pscale_halfs = m->d_pscale ? m->pscale_halfs : 0;
  PinnedBuf pin;
  CU(cudaMallocHost(&pin.p, IO_CHUNK));
  FILE *f = fopen(path, "wb");
  if (!f) return fail(FR_B200_E_ARG, std::string("cannot open ") + path + " for writing");
  int rc = fwrite(&h, sizeof(h), 1, f) == 1 ? 0 : fail(FR_B200_E_ARG, "short write to the packed model file");
  if (!rc) rc = write_blob(f, m->d_weights, h.weights_bytes, pin.p);
  if (!rc) rc = write_blob(f, m->d_rscale, h.rscale_n * 2, pin.p);
  if (!rc) rc = write_blob(f, m->d_vecs, h.vecs_n * 4, pin.p);
  if (!rc) rc = write_blob(f, m->d_emb, h.emb_bytes, pin.p);
  if (!rc) rc = write_blob(f, m->d_qcopy, h.qcopy_bytes, pin.p);
  if (!rc) rc = write_blob(f, m->d_qscale, h.qscale_halfs * 2, pin.p);
  if (!rc) rc = write_blob(f, m->d_pscale, h.pscale_halfs * 2, pin.p);
  if (fclose(f) != 0 && !rc) rc = fail(FR_B200_E_ARG, "closing the packed model file failed");
  return rc;
}

int fr_b200_load_packed(const char *path, int max_batch, int device, int host_visible_state, fr_b200_model **out) {
  if (!path || !out) return fail(FR_B200_E_ARG, "null argument");
  *out = nullptr;
  FILE *f = fopen(path, "rb");
  if (!f) return fail(FR_B200_E_ARG, std::string("cannot open ") + path);
  PackedHeader h;
  if (fread(&h, sizeof(h), 1, f) != 1 || memcmp(h.magic, "FRB200P2", 8) != 0) {
    fclose(f);
    return fail(FR_B200_E_ARG, std::string(path) + " is not a packed model file of this library version");
  }
  fr_b200_config cfg = h.cfg;
  cfg.max_batch = max_batch; cfg.device = device; cfg.host_visible_state = host_visible_state;
  fr_b200_model *m = nullptr;
  // the file decides whether the row copies exist, not this process's environment
  const char *prev = getenv("FR_B200_ROW_COPIES");
  const std::string prev_s = prev ? prev : "";
  setenv("FR_B200_ROW_COPIES", h.has_row_copies || cfg.weight_format == FR_B200_W_FP16 ? "1" : "0", 1);
  int rc = fr_b200_create(&cfg, &m);
  if (prev) setenv("FR_B200_ROW_COPIES", prev_s.c_str(), 1); else unsetenv("FR_B200_ROW_COPIES");
  if (rc) { fclose(f); return rc; }
  const uint64_t emb_bytes = (uint64_t)m->V * m->C * (h.emb_dtype == FR_B200_T_F16 ? 2 : 4);
  if (h.weights_bytes != m->weights_bytes || h.rscale_n != m->rscale_n || h.vecs_n != m->vecs_n || h.emb_bytes != emb_bytes ||
      h.qcopy_bytes != m->qcopy_bytes || h.qscale_halfs != m->qscale_halfs || h.pscale_halfs != m->pscale_halfs ||
      (h.emb_dtype != FR_B200_T_F16 && h.emb_dtype != FR_B200_T_F32)) {
    fclose(f);
    fr_b200_destroy(m);
    return fail(FR_B200_E_ARG, "packed model file does not match this library's layout (written by another version?)");
  }
  PinnedBuf pin;
  cudaError_t ce = cudaMallocHost(&pin.p, IO_CHUNK);
  if (ce == cudaSuccess) ce = cudaMalloc((void **)&m->d_emb, emb_bytes);
  if (ce != cudaSuccess) { fclose(f); fr_b200_destroy(m); return fail(FR_B200_E_NOMEM, cudaGetErrorString(ce)); }
  m->emb_dtype = h.emb_dtype;
  if (!rc) rc = read_blob(f, m->d_weights, h.weights_bytes, pin.p);
  if (!rc) rc = read_blob(f, m->d_rscale, h.rscale_n * 2, pin.p);
  if (!rc) rc = read_blob(f, m->d_vecs, h.vecs_n * 4, pin.p);
  if (!rc) rc = read_blob(f, m->d_emb, h.emb_bytes, pin.p);
  if (!rc) rc = read_blob(f, m->d_qcopy, h.qcopy_bytes, pin.p);
  if (!rc) rc = read_blob(f, m->d_qscale, h.qscale_halfs * 2, pin.p);
  if (!rc) rc = read_blob(f, m->d_pscale, h.pscale_halfs * 2, pin.p);
  fclose(f);
  if (!rc) {
    for (auto &kv : m->mats) kv.second.set = true;
    for (auto &kv : m->vecs) kv.second.set = true;
    m->emb_rows_set.assign(m->V, 1);
    // fp16 models created with their W^T copies (RWKV-5.x, or more than 8 streams) rebuild them from the tiles
    if (m->d_plain) {
      cudaFree(m->d_plain);
      m->d_plain = nullptr;
      rc = ensure_row_copies(m);
    }
  }
  if (!rc) rc = fr_b200_finalize(m);
  if (rc) { fr_b200_destroy(m); return rc; }
  *out = m;
  return FR_B200_OK;
}

int fr_b200_get_config(const fr_b200_model *m, fr_b200_config *cfg) {
  if (!m || !cfg) return fail(FR_B200_E_ARG, "null argument");
  *cfg = m->cfg;
  return FR_B200_OK;
}

int fr_b200_get_info(const fr_b200_model *m, fr_b200_info *info) {
  if (!m || !info) return fail(FR_B200_E_ARG, "null argument");
  info->n_ctas = m->grid; info->n_threads = NTHREADS; info->smem_bytes = (int)m->smem[0]; info->n_stages = m->n_stages[0];
  info->stage_bytes = (int)stage_bytes(m->fmt, kt_max(m->fmt)); info->n_phases = (int)m->phases.size();
  info->weight_stream_bytes = m->stream_bytes; info->launches = m->launches;
  return FR_B200_OK;
}

}  // extern "C"
