// Structures shared by the C-ABI implementation (api.cu), the packers (pack.cu) and the persistent
// decode kernel (decode.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "layout.h"

namespace frb {

constexpr int NW = 8;                       // consumer warps per CTA
constexpr int NCONS = NW * 32;              // consumer threads
constexpr int NTHREADS = NCONS + 128;       // + one producer warp group (one thread of it issues the copies)
constexpr int MAX_STAGES = 12;
constexpr int MAX_B = 8;

// What a phase does around its matvecs.
enum PhaseKind {
  PH_ATT_KVR = 0,   // v4: LN1 + mix -> K,V,R row blocks of the same 16 channels -> WKV update -> r*wkv
  PH_ATT_O = 1,     // v4/v5: output projection + residual
  PH_FFN_KR = 2,    // LN2 + mix -> ffn key (relu^2) and ffn receptance (sigmoid)
  PH_FFN_V = 3,     // ffn value, gated residual, optional x/2
  PH_HEAD = 4,      // ln_out + vocabulary head
  PH5_KVRG = 5,     // v5: LN1 + mix -> K,V,R(,G) row blocks, raw sums (gate through SiLU)
  PH5_WKV = 6,      // v5: per-head state update + readout (no weights)
  PH_MATVEC = 7,    // stand-alone y = W x (unit tests): input vector from kk, output to logits
};

struct PhaseDev {
  const uint8_t *w;        // packed tiles: [item][sub][stage]
  const __half *rscale;    // int8: per-row scales in (item, sub, row) order; else null
  int kind;
  int layer;
  int K;                   // inputs of every matvec of the phase
  int n_items;             // row blocks (all classes together); 0 for PH5_WKV
  int n_sub;               // matrices fused per item (3 for PH_ATT_KVR, else 1)
  int split[3];            // item index where class 1, 2, 3 start (PH_FFN_KR, PH5_KVRG)
  int rot;                 // item i runs on CTA (i + rot) % gridDim.x
  int pad;
  // per-layer vectors the phase's own threads read (saves the hop through the layer table):
  // PH_ATT_KVR, PH5_WKV: time_first, time_decay; PH_ATT_O of RWKV-5: ln_x weight, bias
  const float *aux0, *aux1;
};

// Per-layer vectors (all fp32 on the device) and state offsets.
struct LayerDev {
  const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
  const float *att_mix[4];   // k, v, r, (g)
  const float *ffn_mix[2];   // k, r
  const float *decay, *first;
  const float *lnx_w, *lnx_b;  // v5
};

// One element of an exchange vector (a vector one phase writes and the next phases read across CTAs):
// the fp32 value rounded to 16 significant bits with an 8-bit tag of the writing phase in its low mantissa bits.
// A reader knows which phase must have produced the value and polls until the tag matches, so the data
// is its own synchronisation: no grid-wide barrier, no fence, one 32-bit store per value.
typedef uint32_t exch_t;   // fp32 value, low 8 mantissa bits = tag of the phase that wrote it

struct DecodeParams {
  int version, L, C, F, V, Vpad, H;
  int fmt, act_fp16, rescale_every;
  int B;
  int n_phases;
  int n_stages;
  int l2_prefetch_bytes;       // per CTA: how far ahead of the ring the producer asks L2 for tiles (0 = off)
  unsigned seq_base;           // tag of phase pi of this launch = 1 + (seq_base + pi) % 255; host keeps it >= 255
  unsigned par_mask;           // bit b: which copy of the token-shift states stream b reads (it writes the other)
  int ids_val[MAX_B];
  const unsigned long long *ids_packed;  // when non-null: ids are the packed arg-max words of the previous token
  unsigned long long *amax;    // optional [B]: packed arg-max of this token's logits (zeroed by the host)
  const void *emb;             // [V][C], fp32 when emb_f32 else fp16 (the file's dtype)
  int emb_f32;
  const LayerDev *layers;
  const float *lnout_w, *lnout_b;
  // optional: fp16 image of the whole per-layer vector blob (vecs32 = its fp32 original, same element offsets), given
  // when every LayerNorm weight / bias and token-shift mix vector is exact in fp16; the one-stream kernel then stages
  // these vectors in shared memory as fp16
  const __half *vecs16;
  const float *vecs32;
  const PhaseDev *phases;
  // Residual stream, two copies: x as the ffn value phase (or nothing yet, at layer 0) left it, xa as the attention
  // output phase left it.  A phase never overwrites the copy that CTAs of the phase before it may still be reading.
  exch_t *x, *xa;
  exch_t *rwkv, *kk, *rr;               // [B][C], [B][F], [B][C]
  exch_t *k5, *v5, *r5, *g5, *o5;       // v5 exchange vectors [B][C]
  float *logits;                        // [B][Vpad]
  uint8_t *state;                       // stream slot b at state + b * state_stride
  size_t state_stride, layer_stride;    // bytes
  int *status;                          // 0 = ok, else first failure code
  unsigned long long *prof;             // optional [n_phases][8] profile of CTA 0
};

// status codes written by the kernel
constexpr int ST_TIMEOUT_FULL = 101, ST_TIMEOUT_EMPTY = 102, ST_TIMEOUT_DATA = 103;

// State bytes inside one layer of one stream slot.  The token-shift states exist twice (a token reads
// copy `par` and writes copy `1 - par`), so no CTA can overwrite a value another CTA still has to read.
//   RWKV-4: sx[2][C] act, aa[C], bb[C], pp[C] f32, ffn_sx[2][C] act
//   RWKV-5: sx[2][C] act, s[H][64][64] f32, ffn_sx[2][C] act
FRB_HD size_t act_bytes(int act_fp16) { return act_fp16 ? 2 : 4; }
FRB_HD size_t mid_bytes(int C, int H, int v5) { return v5 ? (size_t)H * 4096 * 4 : 3 * (size_t)C * 4; }
FRB_HD size_t layer_bytes(int C, int H, int v5, int act_fp16) { return 4 * C * act_bytes(act_fp16) + mid_bytes(C, H, v5); }
FRB_HD size_t off_sx(int C, int act_fp16, int par) { return (size_t)par * C * act_bytes(act_fp16); }
FRB_HD size_t off_mid(int C, int act_fp16) { return 2 * (size_t)C * act_bytes(act_fp16); }
FRB_HD size_t off_ffn_sx(int C, int H, int v5, int act_fp16, int par) {
  return off_mid(C, act_fp16) + mid_bytes(C, H, v5) + (size_t)par * C * act_bytes(act_fp16);
}

// ---- seq-mode GEMM (prefill.cu) --------------------------------------------------------------------
enum GemmEpilogue {
  GEMM_EPI_F32 = 0,         // out f32 = acc
  GEMM_EPI_SILU_F16,        // out f16 = acc * sigmoid(acc)
  GEMM_EPI_SIGMOID_F16,     // out f16 = sigmoid(acc)
  GEMM_EPI_RELU2_F16,       // out f16 = max(acc, 0)^2
  GEMM_EPI_ADD_F32,         // out f32 = (aux0 + acc) * scale                (aux0 f32 [M, N])
  GEMM_EPI_MULADD_F32,      // out f32 = (aux0 + aux1 * acc) * scale         (aux1 f16 [M, N])
  GEMM_EPI_PLAIN_F16        // out f16 = acc
};
struct GemmArgs {
  const __half *A;     // [M, K] row-major
  const __half *A2;    // optional [M, K]: low halves of the activations (A + A2 is the fp32 value to ~22 bits)
  const __half *Bt;    // [N, K] row-major (the weight matrix transposed: one row per output channel)
  const __half *Bt2;   // optional [N, K]: what rounding the weights to fp16 lost (int4: q * scale needs 14 bits); third pass
  const __half *col_scale;   // optional [N]: acc *= col_scale[n] before the epilogue (int8: Bt holds the integer codes)
  // quantised weights in packed form instead of Bt (few-row GEMM that expands them in shared memory):
  const uint8_t *Wq;         // wfmt FMT_INT8: codes [N, K] int8;  FMT_INT4: [N, K/2], nibble = q + 8, even k low
  const __half *wq_scale;    // FMT_INT4: group scales [N, K/32] (int8 row scales go in col_scale)
  int wfmt;
  int M, N, K;         // K a multiple of 64
  int epi;
  void *out;           // [M, ldo]
  void *out_lo;        // optional, fp16 epilogues: what rounding out to fp16 lost, same shape
  int ldo;
  const void *aux0, *aux1;   // [M, ldo] like out
  const void *aux1_lo;       // optional: fp16 rounding remainder of aux1
  float scale;
  int *status;         // device word: set when a bounded wait gives up
  float *raw;          // optional scratch [GEMM_SPLIT_MAX][M][N] f32: allows split-K when M <= GEMM_SMALL_M
};
constexpr int GEMM_GROUP_MAX = 4;
constexpr int GEMM_SMALL_M = 1024;    // up to this many rows the GEMM puts the weights along the MMA rows (and splits K, given scratch)
constexpr int GEMM_SPLIT_MAX = 16;
int device_sm_count();   // SMs of the current device
cudaError_t launch_gemm_f16(const GemmArgs &g, cudaStream_t st);   // one GEMM; 256-row tiles when M > 128
// n <= 4 GEMMs with equal M in one launch; mt = 128-row sub-tiles per CTA (1 or 2)
cudaError_t launch_gemm_group(const GemmArgs *probs, int n, int mt, cudaStream_t st, int *defer_split = nullptr);
// row kernels of seq mode
struct SeqLnArgs {
  const float *x;            // [T, C] residual stream
  const float *ln_w, *ln_b;  // [C]
  const float *mix[4];       // nvec mix vectors [C]
  __half *op[4];             // nvec outputs [T, C]
  __half *op_lo[4];          // optional: what the fp16 rounding of op[v] lost (null = not wanted)
  const void *sx_rd;         // shift state read for token 0 (act dtype)
  void *sx_wr;               // shift state written from token T-1
  int T, C, nvec, act_fp16;
  int batch_mode;            // rows are streams: shift states are per row, state_stride bytes apart
  size_t state_stride;
  // optional (pend_split > 1, batch mode): the projection before this LayerNorm has not been finished -- its
  // split-K slabs [pend_split][T][C] are summed here and x = (x + [r *] sum) * pend_scale is stored to x_wr first
  const float *pend_raw;
  const __half *pend_cscale;          // its per-column scales, or null
  const __half *pend_r, *pend_r_lo;   // [T, C] factor of the sum (channel mix), or null (time mix: plain add)
  float pend_scale;
  int pend_split;
  float *x_wr;
};
struct SeqWkvArgs {
  const float *r, *k, *v;    // [T, C]
  const float *decay, *first;  // [H * 64], or [H] when per_head
  float *state;              // [H, 64 key, 64 value], updated in place
  float *y;                  // [T, C]
  int T, C, per_head;
  int n_chunks, chunk_len;   // the sequence is scanned in n_chunks parallel pieces of chunk_len tokens
  float *e_out, *s_in;       // [H, n_chunks, 64, 64] scratch: chunk end states from zero, chunk start states
  int batch_mode;            // rows are streams (T of them, one token each); n_chunks must be 1
  size_t state_stride;       // floats between the states of consecutive streams
};
struct Wkv4Args {
  const float *k, *v, *r;    // [rows, C]; r before the sigmoid
  const float *decay, *first;  // [C]
  void *state;               // aa[C], bb[C], pp[C] of stream 0; state_stride bytes to the next stream
  size_t state_stride;
  __half *out;               // [rows, C] sigmoid(r) * wkv
  __half *out_lo;            // optional: its fp16 rounding remainder
  int T, C, batch_mode;      // seq: T rows of one stream; batch: T streams, one row each
  // optional (split > 1): k, v, r are still split-K slabs [split][T][C] (+ per-column scales), summed in the kernel
  const float *raw_k, *raw_v, *raw_r;
  const __half *cs_k, *cs_v, *cs_r;
  int split;
};
cudaError_t launch_gather_emb(const void *emb, int emb_f32, const int32_t *ids, int T, int C, float *x, cudaStream_t st);
cudaError_t launch_ln_mix_seq(const SeqLnArgs &a, cudaStream_t st);
cudaError_t launch_wkv5_seq(const SeqWkvArgs &a, int H, cudaStream_t st);
int wkv5_scan_slots();   // resident (head, chunk) CTAs of the scan on this device
cudaError_t launch_gn_gate_seq(const float *y, const float *lnx_w, const float *lnx_b, const __half *g, const __half *g_lo, int T,
                               int H, __half *out, __half *out_lo, cudaStream_t st);
cudaError_t launch_wkv4_rows(const Wkv4Args &a, cudaStream_t st);
// device-side Sampler::Sample over the rows of a logits matrix (sample.cu)
size_t sample_scratch_bytes(int rows, int V);
cudaError_t launch_sample_rows(const float *logits, int rows, int V, int ld, float temperature, int top_k, float top_p,
                               const float *u, int32_t *out, void *scratch, size_t scratch_bytes, cudaStream_t st);
cudaError_t launch_logits_add(float *logits, int ld, const int32_t *stream, const int32_t *token, const float *delta, int n, cudaStream_t st);
struct GreedyCtl {           // device-side cursor of a greedy run through the GEMM path
  int32_t *hist;             // [n_tokens][rows] sampled ids
  int step;                  // next row of hist
};
cudaError_t launch_argmax_rows(const float *logits, int rows, int V, int ld, int32_t *out, GreedyCtl *ctl, cudaStream_t st);
cudaError_t launch_ln_row(const float *x, const float *w, const float *b, int C, float *out, cudaStream_t st);
cudaError_t launch_transpose_f16(const __half *src, int K, int N, __half *dst, cudaStream_t st);   // [K,N] -> [N,K]

// ---- launchers implemented in the .cu files ------------------------------------------------------
// mode = how many streams one launch carries: 0 -> 1, 1 -> up to 4, 2 -> up to 8
inline int decode_mode(int batch) { return batch == 1 ? 0 : batch <= 4 ? 1 : 2; }
// par16: the launch will carry DecodeParams::vecs16 (LayerNorm parameters staged as fp16)
size_t decode_smem_bytes(int fmt, int mode, int C, int F, int version, int n_stages, int par16 = 0);
cudaError_t launch_decode(const DecodeParams &p, int mode, int grid, size_t smem, cudaStream_t st);
cudaError_t decode_max_grid(int fmt, int mode, size_t smem, int device, int *grid);
// packed arg-max word = {order-preserving image of the fp32 logit, 0xFFFFFFFF - index}: a 64-bit max picks the
// largest logit and, among equals, the smallest index
cudaError_t launch_unpack_ids(const unsigned long long *packed, int n, int32_t *out, cudaStream_t st);
cudaError_t launch_wait_selftest(int *status, unsigned long long limit_ns, cudaStream_t st);

// quantise / pack (pack.cu); all pointers device
cudaError_t launch_f16_to_f32(const __half *src, float *dst, size_t n, cudaStream_t st);
cudaError_t launch_f32_to_f16(const float *src, __half *dst, size_t n, cudaStream_t st);
cudaError_t launch_i8_to_f16(const int8_t *src, __half *dst, size_t n, cudaStream_t st);
cudaError_t launch_f32_split_f16(const float *src, __half *hi, __half *lo, size_t n, cudaStream_t st);
cudaError_t launch_quant_int8(const float *W, int K, int N, int8_t *q, __half *scales, cudaStream_t st);
cudaError_t launch_quant_int4(const float *W, int K, int N, uint8_t *packed, __half *scales, cudaStream_t st);
cudaError_t launch_dequant_int8(const int8_t *q, const __half *scales, int K, int N, float *W, cudaStream_t st);
cudaError_t launch_dequant_int4(const uint8_t *packed, const __half *scales, int K, int N, float *W, cudaStream_t st);
// Pack one matrix into tiles.  src depends on fmt: fp16 -> __half W[K][N]; int8 -> q[N][K] (+scales[N]);
// int4 -> packed[N][K/2] (+scales[N][K/32]).  Row block rb of the matrix goes to dst + rb * item_stride.
// rscale_dst (int8): per-row scales, row r of block rb at rscale_dst[rb * rscale_stride + r].
cudaError_t launch_pack(int fmt, const void *src, const __half *scales, int K, int N, uint8_t *dst,
                        size_t item_stride, __half *rscale_dst, size_t rscale_stride, cudaStream_t st);
// Inverse of launch_pack: tiles -> dequantised fp32 W[K][N].
cudaError_t launch_unpack(int fmt, const uint8_t *tiles, size_t item_stride, const __half *rscale,
                          size_t rscale_stride, int K, int N, float *W, cudaStream_t st);

}  // namespace frb
