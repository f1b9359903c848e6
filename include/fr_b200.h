/*
 * fr_b200 — C ABI of the B200 (sm_100a) RWKV forward backend.
 *
 * This is the boundary the registry glue (faster-rwkv_b200/backend/registry_backend.cpp)
 * and the ctypes host mirror (faster-rwkv_b200/__init__.py) bind.  Each entry point names
 * the piece of the reference (daquexian/faster-rwkv, path:line inside that tree) it replaces.
 *
 * Conventions
 *   - every function returns 0 (FR_B200_OK) or a negative status; none throws, none aborts;
 *     fr_b200_strerror() turns a status into text and fr_b200_last_error() gives detail;
 *   - pointers marked "host or device" are copied with cudaMemcpyDefault (unified addressing);
 *   - matrices are given exactly as the reference's `.fr` file stores them: row-major
 *     [in, out] (kernels/cuda/matmul.cpp:105-122), fp16 or fp32;
 *   - all GPU work of a model runs on the stream passed to the call (0 = default stream);
 *   - a model belongs to one device and one host thread at a time (the reference's Model is
 *     single-threaded as well, kernels/registry.h:11-35).
 */
#ifndef FR_B200_H_
#define FR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fr_b200_model fr_b200_model;

enum {
  FR_B200_OK = 0,
  FR_B200_E_ARG = -1,          /* bad argument (null pointer, shape, range) */
  FR_B200_E_UNSUPPORTED = -2,  /* model shape / version / batch not supported */
  FR_B200_E_CUDA = -3,         /* a CUDA runtime call failed */
  FR_B200_E_STATE = -4,        /* call order (e.g. decode before finalize) */
  FR_B200_E_MISSING = -5,      /* finalize: a tensor of the model was never set */
  FR_B200_E_TIMEOUT = -6,      /* a bounded device-side wait gave up; results are invalid */
  FR_B200_E_NOMEM = -7
};

/* weight formats = the reference's strategy dtype strings (model.cpp:44-60) */
enum { FR_B200_W_FP16 = 0, FR_B200_W_INT8 = 1, FR_B200_W_INT4 = 2 };
/* tensor element types accepted by fr_b200_set_tensor (tensor.h:33-41) */
enum { FR_B200_T_F16 = 0, FR_B200_T_F32 = 1 };
/* model versions = the `.fr` "version" string (kernels/default/init_model.cpp:58-73) */
enum { FR_B200_V4 = 4, FR_B200_V5_0 = 50, FR_B200_V5_1 = 51, FR_B200_V5_2 = 52 };

typedef struct fr_b200_config {
  int version;        /* FR_B200_V4 ... */
  int n_layer;
  int n_embd;         /* multiple of 64 */
  int n_ffn;          /* multiple of 64 */
  int n_head;         /* RWKV-5 only (head size must be 64), else 0 */
  int vocab;
  int weight_format;  /* FR_B200_W_* */
  int act_fp16;       /* 1: "cuda fp16" semantics — fp16 token-shift states and x /= 2 every 6 layers
                         (kernels/default/model_forward.cpp:173-175); 0: fp32 activations ("int8"/"int4") */
  int max_batch;      /* stream slots, 1..4096.  Up to 8 streams per call run in the persistent kernel; a model created
                       * with max_batch > 8 also keeps every projection as fp16 W^T (dequantised for int8 / int4) and
                       * decodes larger batches through tensor-core GEMMs, one row per stream */
  int device;         /* CUDA device ordinal */
} fr_b200_config;

/* ---- model life cycle: replaces def::init_model (kernels/default/init_model.cpp:19-133) ---- */

/* Allocate a model on cfg->device.  Nothing is uploaded yet. */
int fr_b200_create(const fr_b200_config *cfg, fr_b200_model **out);

/* Give one tensor under its `.fr` name ("blocks.3.att.key.weight", "ln_out.bias", "emb.weight" as
 * one [vocab, n_embd] array or "emb.<row>" per row as init_model.cpp:128-132 holds them).
 * data: host or device.  Matrices are repacked to the streaming tile layout (and quantised when the
 * model's weight_format is int8 / int4) on the GPU during this call. */
int fr_b200_set_tensor(fr_b200_model *m, const char *name, const void *data, int dtype,
                       const int64_t *shape, int ndim);

/* Check that every tensor arrived, build the phase table, reset all streams' states. */
int fr_b200_finalize(fr_b200_model *m);

void fr_b200_destroy(fr_b200_model *m);

/* ---- forward: replaces def::ModelForward (kernels/default/model_forward.cpp:22-193) and the
 * kernels it calls: layer_norm_op (kernels/cuda/layer_norm.cu:101-130), Mix / FfnOneMix
 * (kernels/cuda/att.cu:90-143, ffn.cu:15-32), gemm_cublas_tensor (kernels/cuda/matmul.cpp:105-122),
 * WkvForwardOne (att.cu:30-62), OneV5MulAdd + group_norm_op (att.cu:64-81, group_norm.cu:322-357),
 * InplaceSigmoid / InplaceReLUAndSquare / InplaceFma (ffn.cu:34-60), cast_dtype (cast_dtype.cu:24-41).
 *
 * One token for each of `batch` independent streams (stream b uses state slot b).
 * ids: host, [batch].  logits: host or device, [batch, vocab] fp32, or NULL.
 * argmax: host or device, [batch] int32 (greedy sample, Sampler::Sample top_k=1, sampler.cpp:71-74), or NULL.
 * Synchronous with respect to the host when logits or argmax is a host pointer. */
int fr_b200_decode(fr_b200_model *m, const int32_t *ids, int batch, float *logits, int32_t *argmax,
                   void *stream);

/* Greedy generation that never returns to the host between tokens: token t+1 of stream b is the argmax
 * of stream b's logits at step t, taken on the device (replaces the Run -> D2H -> Sampler::Sample(top_k=1)
 * round trip of chat.cpp:60-95 / sampler.cpp:71-74).  first_ids: host [batch].  out_ids: host or device,
 * [n_tokens, batch] — the sampled ids (row t = the tokens chosen after step t). */
int fr_b200_decode_greedy(fr_b200_model *m, const int32_t *first_ids, int batch, int n_tokens, int32_t *out_ids,
                          void *stream);

/* Sampler::Sample (sampler.cpp:38-101) on the device, over the logits the last decode of `batch` streams left there:
 * softmax, descending sort, top_p prefix, top_k cut, probs^(1/temperature) with temperature clamped to [0.1, 5],
 * inverse-CDF draw.  uniform: host [batch], the draw in [0, 1] of each stream -- the reference computes it as
 * (g() - g.min()) / (g.max() - g.min()) from a std::minstd_rand0 (sampler.cpp:20-22); a host that does the same gets
 * the reference's choice.  ids: host or device [batch].  No [V] logits cross to the host, no host sort. */
int fr_b200_sample(fr_b200_model *m, int batch, float temperature, int top_k, float top_p, const float *uniform,
                   int32_t *ids, void *stream);

/* Device pointer of the [max_batch, vocab_padded] fp32 logits of the last decode (row stride =
 * fr_b200_vocab_padded()); valid until the next decode. */
int fr_b200_logits_device(fr_b200_model *m, float **ptr);
int fr_b200_vocab_padded(const fr_b200_model *m);

/* Seq mode = the token loop of kernels/default/model_forward_seq.cpp:34-46 on stream slot `slot`:
 * feeds n ids in order, writes the last token's logits. */
int fr_b200_run_seq(fr_b200_model *m, int slot, const int32_t *ids, int n, float *last_logits, void *stream);

/* ---- recurrent state: replaces Model::ResetStates (model.cpp:145-177) and the state tensors the
 * layer loop assigns (model_forward.cpp:112-117).  Layout per stream slot, per layer:
 *   RWKV-4: sx[C] act, aa[C] f32, bb[C] f32, pp[C] f32, ffn_sx[C] act          (model.cpp:149-162)
 *   RWKV-5: sx[C] act, s[H,64,64] f32 (key-major), ffn_sx[C] act               (model.cpp:163-175)
 * "act" is fp16 when act_fp16 else fp32. */
int fr_b200_state_reset(fr_b200_model *m, int slot);                 /* slot -1 = all */
int fr_b200_state_count(const fr_b200_model *m);                     /* tensors per layer: 5 or 3 */
/* Device address, element type (FR_B200_T_*) and element count of state tensor (slot, layer, index). */
int fr_b200_state_tensor(fr_b200_model *m, int slot, int layer, int index, void **dev_ptr, int *dtype,
                         int64_t *numel);
int fr_b200_state_export(fr_b200_model *m, int slot, void *dst, size_t dst_bytes); /* dst host or device */
int fr_b200_state_import(fr_b200_model *m, int slot, const void *src, size_t src_bytes);
size_t fr_b200_state_bytes(const fr_b200_model *m);                  /* bytes of one slot */

/* ---- quantisers (new formats; the reference's own int8/int4 exist only for its ncnn exporter,
 * kernels/export-ncnn/kernels.cpp:253-592).  W: [K,N] fp32, host or device.
 * int8: q [N,K] int8, scales [N] fp16, scale = fp16(max_k|W|/127), q = clamp(round_half_away(W/scale)).
 * int4: packed [N,K/2] (nibble = q+8, even k in the low nibble), scales [N,K/32] fp16 = fp16(max|W|/7).
 * Outputs are host or device.  The *_dequant functions return the [K,N] fp32 matrix. */
int fr_b200_quantize_int8(const float *W, int K, int N, int8_t *q, uint16_t *scales, int device);
int fr_b200_quantize_int4(const float *W, int K, int N, uint8_t *packed, uint16_t *scales, int device);
int fr_b200_dequantize_int8(const int8_t *q, const uint16_t *scales, int K, int N, float *W, int device);
int fr_b200_dequantize_int4(const uint8_t *packed, const uint16_t *scales, int K, int N, float *W, int device);

/* Unpack one matrix of a finalized model from its streaming tiles back to [K,N] fp32 (dequantised).
 * name = the `.fr` name.  For bit-exactness tests of the tile packing. */
int fr_b200_unpack_matrix(fr_b200_model *m, const char *name, float *W, int K, int N);

/* ---- single kernels, for unit tests (each replaces the reference kernel named beside it) ---- */

/* y[batch,N] = x[batch,K] @ W  with W given as [K,N] fp32 and run through the given weight format:
 * replaces gemm_cublas_tensor for the m=1 case (kernels/cuda/matmul.cpp:105-122). x,y host or device fp32. */
int fr_b200_matvec(const float *W, int K, int N, int weight_format, const float *x, int batch, float *y,
                   int device);

/* The same matvec for callers that are not allowed to allocate (no counterpart in the reference; it allocates
 * through its caching allocator on every op, kernels/cuda/allocator.cpp:47-479).  Meant for hosts that fix their
 * GPU memory budget up front — a serving process whose execute callback must not call cudaMalloc, which stalls the
 * whole device and may fail once a framework pool owns the memory, or a latency-bound loop.  All scratch (the
 * converted matrix, the packed tiles, scales, padded output, descriptor) sits in a fixed 4.7 MiB array inside the
 * library image, present on every GPU that loads the library until the process ends.
 *   - W [K,N], x [batch,K], y [batch,N]: fp32 DEVICE pointers on `device`; x must be 16-byte aligned (the kernel
 *     reads it in place with 16-byte loads; FR_B200_E_ARG otherwise); nothing is allocated, no
 *     cudaMalloc / cudaFree / pool routine is called.
 *   - limits: K a multiple of 64, K <= 8192, N <= 16384, ceil16(N) * K <= 1,048,576, batch <= 8; larger inputs
 *     return FR_B200_E_UNSUPPORTED with the reason in fr_b200_noalloc_last_error().
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress); make it before any
 *     stream capture begins.  Every call copies a status word back and synchronises `stream`, so it must never be
 *     made on a capturing stream (FR_B200_E_STATE), and not again after the device's context was reset.
 *   - every call reuses the one array: calls whose GPU work can overlap race; serialise them.
 * Synchronises `stream` before returning. */
int fr_b200_matvec_noalloc(const float *W, int K, int N, int weight_format, const float *x, int batch, float *y,
                           int device, void *stream);
const char *fr_b200_noalloc_last_error(void);

/* out[M,N] = epilogue(A[M,K] @ W[K,N]) on the tcgen05 tensor cores, fp16 operands, fp32 accumulate: the seq-mode
 * replacement of gemm_cublas_tensor (kernels/cuda/matmul.cpp:105-122) with the element-wise kernels that follow
 * it in the reference fused as the epilogue (att_seq.cu:368-423, ffn_seq.cu:65-87).  A: [M,K] fp32, rounded to
 * fp16; W: [K,N] fp32, rounded to fp16; out, aux0, aux1: [M,N] fp32, host or device.  K a multiple of 64.
 * epilogue: 0 acc | 1 silu(acc) | 2 sigmoid(acc) | 3 relu(acc)^2 | 4 (aux0 + acc) * scale |
 *           5 (aux0 + aux1 * acc) * scale | 6 acc rounded to fp16.   For unit tests. */
int fr_b200_gemm_f16(const float *A, const float *W, int M, int N, int K, int epilogue, const float *aux0,
                     const float *aux1, float scale, float *out, int device);

/* ---- introspection ---- */
typedef struct fr_b200_info {
  int n_ctas, n_threads, smem_bytes, n_stages, stage_bytes, n_phases;
  long long weight_stream_bytes;   /* bytes of packed weights one token streams (algorithmic bytes) */
  long long launches;              /* kernels launched by this model so far */
} fr_b200_info;
int fr_b200_get_info(const fr_b200_model *m, fr_b200_info *info);

/* One decode step with a per-CTA, per-phase trace: stamps[cta][phase][8] = {phase start, inputs staged, row
 * blocks done (ns of the GPU's global timer), then SM cycles: waiting for weight tiles, phase descriptor ->
 * phase start, phase start -> inputs arrived, inputs arrived -> statistics / conversion done, -> operands staged};
 * zero where the CTA had no work in the phase.
 * A tracing aid (the reference has only wall-clock FR_SHOW_SPEED prints, chat.cpp:98-111).
 * stamps: host, n_ctas * n_phases * 8 entries (fr_b200_get_info gives both counts). */
int fr_b200_decode_profile(fr_b200_model *m, const int32_t *ids, int batch, uint64_t *stamps, int n_stamps);

/* Runs out one bounded device-side wait on purpose, without hanging anything: a one-CTA kernel waits, through the
 * helper every kernel of this library waits with, on a barrier that nothing arrives at, with a limit of limit_us
 * microseconds (1 .. 1,000,000) instead of the built-in 2 s.  The wait gives up, records its status word and the
 * kernel ends normally; the call returns FR_B200_E_TIMEOUT (the expected result) and the context stays usable.
 * The reference has no device-side waits and reports failures as exceptions from CUDA_CHECK (check.h:40-48). */
int fr_b200_wait_selftest(int device, unsigned limit_us);

const char *fr_b200_strerror(int status);
const char *fr_b200_last_error(void);   /* thread-local detail of the last failure */

#ifdef __cplusplus
}
#endif
#endif /* FR_B200_H_ */
