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
  int max_batch;      /* stream slots, 1..4096.  Up to 8 streams per call run in the persistent kernel where its shared
                       * memory can hold their activation vectors (up to 4 at n_ffn = 8192); larger batches are decoded
                       * by tensor-core GEMMs, one row per stream.  For that path fp16 models created with
                       * max_batch > 8 (or too wide for max_batch streams in the persistent kernel) keep every
                       * projection a second time as fp16 W^T; int8 / int4 models always keep a row-major copy of the
                       * packed codes, the same bytes again, which the GEMM expands in shared memory */
  int device;         /* CUDA device ordinal */
  int host_visible_state; /* 1: the recurrent state lives in managed memory, so the device addresses fr_b200_state_tensor
                           * hands out can also be read by the host between calls.  The reference's Model::SaveStateFile
                           * copies the state tensors with a plain memcpy (model.cpp:110); the registry glue sets this so
                           * that the unchanged class can save a CUDA model's state.  0: ordinary device memory. */
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

/* Packed model files: everything fr_b200_finalize left on the device (the streaming tiles, already quantised for
 * int8 / int4; row scales; per-layer vectors; the embedding table; the row-major packed copies) written back to back
 * behind a header.  fr_b200_load_packed brings a model back with a few large reads and copies -- no msgpack parse, no
 * upload per embedding row, no re-quantisation, which is what def::init_model does on every start
 * (kernels/default/init_model.cpp:19-52, 128-132).  The weight format, version and shape come from the file;
 * max_batch, device and host_visible_state are the caller's.  A file written by a library with another tile layout is
 * refused (FR_B200_E_ARG).  The loaded model is finalized. */
int fr_b200_save_packed(fr_b200_model *m, const char *path);
int fr_b200_load_packed(const char *path, int max_batch, int device, int host_visible_state, fr_b200_model **out);
/* The configuration a model was created with (for a model that came from a packed file: the file's). */
int fr_b200_get_config(const fr_b200_model *m, fr_b200_config *cfg);

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

/* logits[streams[i]][tokens[i]] += deltas[i] for i < n, on the logits the last decode left on the device: the sparse
 * adjustments a chat loop makes before it samples -- frequency / presence penalties and the end-of-text / newline
 * biases of chat.cpp:57-75 -- so that sampling can stay on the device.  streams, tokens, deltas: host arrays. */
int fr_b200_logits_add(fr_b200_model *m, int n, const int32_t *streams, const int32_t *tokens, const float *deltas, void *stream);

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

/* ---- stand-alone operators over DEVICE pointers: the forward pass as the reference's operator API cuts it
 * (kernels/kernels.h:15-257).  The decode kernel and the seq path fuse all of these; the entry points below exist so
 * that every formula can be tested and registered on its own (backend/registry_backend.cpp registers the reference's
 * op-level keys "att", "ffn", "layernorm", ... over them).  Tensor element types are FR_B200_T_F16 / FR_B200_T_F32;
 * stream = cudaStream_t (0 = default); calls are asynchronous on that stream unless noted. */

/* LayerNorm of `rows` rows of C elements (eps 1e-5, fp32 statistics: layer_norm_op, kernels/cuda/layer_norm.cu:101-130)
 * and, with nvec > 0, the token-shift mix that follows it in the reference (Mix / MixWithG, kernels/cuda/att.cu:90-143;
 * FfnOneMix, ffn.cu:15-32): out[v] = xx * mix[v] + sx * (1 - mix[v]).  x, sx, xx: act_dtype; ln_w, ln_b, mix[v]:
 * param_dtype; out[v]: out_dtype.  xx may be NULL when only the mixed vectors are wanted; nvec = 0 is a plain LayerNorm. */
int fr_b200_ln_mix(const void *x, const void *sx, const void *ln_w, const void *ln_b, const void *const *mix, int nvec, int rows,
                   int C, int act_dtype, int param_dtype, int out_dtype, void *xx, void *const *out, void *stream);

/* One RWKV-4 WKV step over C channels: WkvForwardOne with the sigmoid gate (kernels/cuda/att.cu:30-62, 154-159).
 * k, v, r (r before the sigmoid), decay (= -exp(raw)), first, aa, bb, pp: fp32 [C].  out = sigmoid(r) * wkv in out_dtype;
 * aa2, bb2, pp2: the new state (may alias the old one). */
int fr_b200_wkv4_step(const float *k, const float *v, const float *r, const float *decay, const float *first, const float *aa,
                      const float *bb, const float *pp, int C, int out_dtype, void *out, float *aa2, float *bb2, float *pp2,
                      void *stream);

/* One RWKV-5 state step over n_head heads of size 64: OneV5MulAdd and the readout around it (kernels/cuda/att.cu:64-81,
 * 219-335).  r, k, v: fp32 [n_head * 64]; decay (= exp(-exp(raw))), first: fp32 [n_head] when per_head (RWKV-5.0) else
 * [n_head * 64]; s, s2: fp32 [n_head, 64 key, 64 value] (s2 must not alias s); y: fp32 [n_head * 64] before GroupNorm. */
int fr_b200_wkv5_step(const float *r, const float *k, const float *v, const float *decay, const float *first, int per_head,
                      const float *s, int n_head, float *s2, float *y, void *stream);

/* The RWKV-5 state recurrence over T tokens as a chunk-parallel scan: replaces rwkv5_2_kernel_forward
 * (kernels/cuda/att_seq.cu:258-345), which walks T serially.  r, k, v, y: fp32 [T, n_head * 64]; state: fp32
 * [n_head, 64, 64], updated in place; n_chunks = parallel pieces (1 = serial).  Synchronises the stream. */
int fr_b200_wkv5_chunk_scan(const float *r, const float *k, const float *v, const float *decay, const float *first, int per_head,
                            float *state, int n_head, int T, int n_chunks, float *y, void *stream);

/* GroupNorm over the last dimension cut into num_groups pieces, eps 1e-5 (group_norm_op, kernels/cuda/group_norm.cu:322-357).
 * x, out: [rows, C] in x_dtype; w, b: [C] in param_dtype. */
int fr_b200_groupnorm(const void *x, const void *w, const void *b, int rows, int C, int num_groups, int x_dtype, int param_dtype,
                      void *out, void *stream);

/* Element-wise pieces (kernels/cuda/att.cu:145-175, ffn.cu:34-60, cast_dtype.cu:24-41, element_wise.cu:15-19, fill.cu:17-26):
 * out[i] = f(x[i], y[i], z[i]) over n elements, each operand with its own element type. */
enum {
  FR_B200_EW_COPY = 0,     /* x (a dtype cast when the types differ) */
  FR_B200_EW_FILL = 1,     /* alpha */
  FR_B200_EW_SCALE = 2,    /* x * alpha (scalar_div_ with alpha = 1 / d) */
  FR_B200_EW_ADD = 3,      /* x + y */
  FR_B200_EW_MUL = 4,      /* x * y */
  FR_B200_EW_SIGMOID = 5,
  FR_B200_EW_RELU2 = 6,    /* max(x, 0)^2 */
  FR_B200_EW_SILU = 7,
  FR_B200_EW_FMA = 8       /* x * y + z */
};
int fr_b200_elementwise(int op, const void *x, int x_dtype, const void *y, int y_dtype, const void *z, int z_dtype, float alpha,
                        void *out, int out_dtype, size_t n, void *stream);
/* out[M,N] = a[M,K] @ w[K,N] over device tensors of either element type: gemm_cublas_tensor (kernels/cuda/matmul.cpp:105-146)
 * for the operator API.  w is rounded to fp16 if it is not already; up to 8 rows run the streaming matvec (the rows
 * travel as fp16 hi + lo pairs), more rows the tensor-core GEMM (rows rounded to fp16).  The matrix is repacked on
 * every call, so this is the operator-level path, not the model's.  K a multiple of 64.  Synchronises the stream. */
int fr_b200_matmul(const void *a, int a_dtype, int M, int K, const void *w, int w_dtype, int N, void *out, int out_dtype,
                   int device, void *stream);
const char *fr_b200_op_last_error(void);

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
