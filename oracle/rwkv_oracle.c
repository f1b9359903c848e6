/*
 * CPU fp32 restatement of the reference's RWKV forward pass and of the weight
 * quantisers.  TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA path and
 * the timed CPU baseline; no product code path may call into it.
 *
 * Every function cites the reference file:line it follows (paths inside the
 * daquexian/faster-rwkv tree).  The reference registers its op compositions
 * (kernels/default/att.cpp, ffn.cpp) only for the ONNX meta device, so there is no
 * upstream "cpu fp32" forward to call; this file restates those compositions with
 * plain fp32 loops.  Parity pin: tests compare it with the reference's own
 * model.cpp + kernels/default/* compiled for the CPU (oracle/_ref) and with golden
 * vectors that binary produced (tests/golden).  The int8 / int4 formats are new
 * (the reference has no CUDA quantised path), so for them parity is unpinned in
 * the reference and this file is the definition.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
  int version;        /* 4, 50 (v5.0), 51 (v5.1), 52 (v5.2) */
  int n_layer, n_embd, n_ffn, n_head, vocab;
  int rescale_every;  /* 6 when the activations are fp16 (model_forward.cpp:173), else 0 */
  int state_fp16;     /* 1: token-shift states are stored as fp16, as under "cuda fp16" where the state
                         tensors have the activation dtype (model.cpp:149-151, kernels/cuda/att.cu:337-359) */
  int gate_from_xx;   /* 1: v5.1/5.2 gate = silu(xx @ Wg) as kernels/default/att.cpp:101 writes it; 0 (default):
                         silu(gx @ Wg) as the CUDA path computes it (kernels/cuda/att.cu:289) */
} orc_cfg;

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

static uint16_t f32_to_f16(float f);
static float f16_to_f32(uint16_t h);
static inline float state_round(float v, int state_fp16) { return state_fp16 ? f16_to_f32(f32_to_f16(v)) : v; }

/* ---------------------------------------------------------------- primitives */

/* LayerNorm over one row, eps 1e-5, biased variance (kernels/cuda/layer_norm.cu:101-130,
 * epsilon at :113; kernels/cuda/group_norm.cu:338 uses the same for GroupNorm). */
static void layernorm(const float *x, const float *g, const float *b, int n, float *y) {
  double mean = 0, var = 0;
  for (int i = 0; i < n; ++i) mean += x[i];
  mean /= n;
  for (int i = 0; i < n; ++i) { double d = x[i] - mean; var += d * d; }
  var /= n;
  float inv = (float)(1.0 / sqrt(var + 1e-5));
  float m = (float)mean;
  for (int i = 0; i < n; ++i) y[i] = (x[i] - m) * inv * g[i] + b[i];
}

/* y[N] = x[K] . W[K,N], W row-major [in,out] (kernels/cuda/matmul.cpp:105-122: fp32
 * accumulate, one rounding of the output). */
static void matvec(const float *x, const float *W, int K, int N, float *y) {
#pragma omp parallel
  {
    int nt = 1, tid = 0;
#ifdef _OPENMP
    nt = omp_get_num_threads(); tid = omp_get_thread_num();
#endif
    /* each thread owns a contiguous block of output columns, 16-aligned */
    int per = ((N + nt - 1) / nt + 15) & ~15;
    int n0 = tid * per, n1 = n0 + per < N ? n0 + per : N;
    if (n0 < n1) {
      for (int n = n0; n < n1; ++n) y[n] = 0.f;
      for (int k = 0; k < K; ++k) {
        const float xv = x[k];
        const float *w = W + (size_t)k * N;
        for (int n = n0; n < n1; ++n) y[n] += xv * w[n];
      }
    }
  }
}

static inline float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

/* kx = xx*mix + sx*(1-mix)  (kernels/default/att.cpp:24-26, ffn.cpp:15-16) */
static void mix(const float *xx, const float *sx, const float *m, int n, float *out) {
  for (int i = 0; i < n; ++i) out[i] = xx[i] * m[i] + sx[i] * (1.f - m[i]);
}

/* ---------------------------------------------------------------- time mix */

/* One WKV step over C channels, kernels/default/att.cpp:30-41 (WkvForwardOne, kernels/cuda/att.cu:30-62, with the
 * sigmoid of att.cu:154-159): out = sigmoid(r) * wkv; aa, bb, pp updated in place.  Exported for per-kernel tests. */
void orc_wkv4_step(int C, const float *k, const float *v, const float *r, const float *decay, const float *first,
                   float *aa, float *bb, float *pp, float *out) {
  for (int i = 0; i < C; ++i) {
    float rr = sigmoidf_(r[i]);
    float ww = first[i] + k[i];
    float pm = pp[i] > ww ? pp[i] : ww;
    float e1 = expf(pp[i] - pm), e2 = expf(ww - pm);
    float wkv = (e1 * aa[i] + e2 * v[i]) / (e1 * bb[i] + e2);
    ww = decay[i] + pp[i];
    pm = ww > k[i] ? ww : k[i];
    e1 = expf(ww - pm);
    e2 = expf(k[i] - pm);
    aa[i] = e1 * aa[i] + e2 * v[i];
    bb[i] = e1 * bb[i] + e2;
    pp[i] = pm;
    out[i] = rr * wkv;
  }
}

/* One RWKV-5 state step over H heads of size S, kernels/default/att.cpp:62-72 / 96-106 (OneV5MulAdd, kernels/cuda/att.cu:64-81):
 * out[h,j] = sum_i r_i (u_i k_i v_j + s_ij), s_ij = k_i v_j + w_i s_ij; decay / first per head when per_head (v5.0).
 * out is the readout before GroupNorm.  Exported for per-kernel tests. */
void orc_wkv5_step(int H, int S, int per_head, const float *r, const float *k, const float *v, const float *decay,
                   const float *first, float *s, float *out) {
  for (int h = 0; h < H; ++h) {
    float *sh = s + (size_t)h * S * S;
    for (int j = 0; j < S; ++j) out[h * S + j] = 0.f;
    for (int i = 0; i < S; ++i) {
      const float u = per_head ? first[h] : first[h * S + i];
      const float w = per_head ? decay[h] : decay[h * S + i];
      const float ki = k[h * S + i], ri = r[h * S + i];
      for (int j = 0; j < S; ++j) {
        float a = ki * v[h * S + j];
        out[h * S + j] += ri * (u * a + sh[i * S + j]);
        sh[i * S + j] = a + w * sh[i * S + j];
      }
    }
  }
}

/* LayerNorm of one row, exported for per-kernel tests (GroupNorm = this over each group). */
void orc_layernorm(const float *x, const float *g, const float *b, int n, float *y) { layernorm(x, g, b, n, y); }

/* RWKV-4 time mix, kernels/default/att.cpp:16-45 (same maths as WkvForwardOne,
 * kernels/cuda/att.cu:30-62).  state: sx, aa, bb, pp each [C], updated in place. */
static void att_v4(int C, int sf16, float *x, float *sx, float *aa, float *bb, float *pp, const float *const *p,
                   float *tmp) {
  const float *ln_w = p[0], *ln_b = p[1], *mk = p[2], *mv = p[3], *mr = p[4], *decay = p[5],
              *first = p[6], *kw = p[7], *vw = p[8], *rw = p[9], *ow = p[10];
  float *xx = tmp, *kx = tmp + C, *vx = tmp + 2 * C, *rx = tmp + 3 * C, *k = tmp + 4 * C,
        *v = tmp + 5 * C, *r = tmp + 6 * C, *out = tmp + 7 * C;
  layernorm(x, ln_w, ln_b, C, xx);
  mix(xx, sx, mk, C, kx);
  mix(xx, sx, mv, C, vx);
  mix(xx, sx, mr, C, rx);
  matvec(rx, rw, C, C, r);
  matvec(kx, kw, C, C, k);
  matvec(vx, vw, C, C, v);
  orc_wkv4_step(C, k, v, r, decay, first, aa, bb, pp, r);
  matvec(r, ow, C, C, out);
  for (int i = 0; i < C; ++i) { x[i] += out[i]; sx[i] = state_round(xx[i], sf16); }
}

/* RWKV-5 / 5.1 / 5.2 one-token time mix: kernels/default/att.cpp:47-113 with the gate fed
 * by gx as the CUDA path does (kernels/cuda/att.cu:289).  State s is [H][S key][S value];
 * decay / first are indexed per head (v5.0, att.cu:242) or per (head, key) (v5.1/5.2,
 * att.cu:306).  GroupNorm with H groups, eps 1e-5 (kernels/cuda/group_norm.cu:322-357). */
static void att_v5(int version, int C, int H, int sf16, int gate_xx, float *x, float *sx, float *s, const float *const *p,
                   float *tmp) {
  const int S = C / H, gate = version >= 51;
  int q = 0;
  const float *ln_w = p[q++], *ln_b = p[q++], *lx_w = p[q++], *lx_b = p[q++], *mk = p[q++],
              *mv = p[q++], *mr = p[q++];
  const float *mg = gate ? p[q++] : NULL;
  const float *decay = p[q++], *first = p[q++], *kw = p[q++], *vw = p[q++], *rw = p[q++];
  const float *gw = gate ? p[q++] : NULL;
  const float *ow = p[q++];
  float *xx = tmp, *kx = tmp + C, *vx = tmp + 2 * C, *rx = tmp + 3 * C, *k = tmp + 4 * C,
        *v = tmp + 5 * C, *r = tmp + 6 * C, *out = tmp + 7 * C, *g = tmp + 8 * C, *gx = tmp + 9 * C;
  layernorm(x, ln_w, ln_b, C, xx);
  mix(xx, sx, mk, C, kx);
  mix(xx, sx, mv, C, vx);
  mix(xx, sx, mr, C, rx);
  matvec(rx, rw, C, C, r);
  matvec(kx, kw, C, C, k);
  matvec(vx, vw, C, C, v);
  if (gate) {
    mix(xx, sx, mg, C, gx);
    matvec(gate_xx ? xx : gx, gw, C, C, g);
    for (int i = 0; i < C; ++i) g[i] = g[i] * sigmoidf_(g[i]); /* SiLU, att.cu:145-152 */
  }
  orc_wkv5_step(H, S, version == 50, r, k, v, decay, first, s, out);
  for (int h = 0; h < H; ++h) layernorm(out + h * S, lx_w + h * S, lx_b + h * S, S, out + h * S);
  if (gate) for (int i = 0; i < C; ++i) out[i] *= g[i];
  matvec(out, ow, C, C, k /* reuse */);
  for (int i = 0; i < C; ++i) { x[i] += k[i]; sx[i] = state_round(xx[i], sf16); }
}

/* Channel mix, kernels/default/ffn.cpp:8-23. */
static void ffn(int C, int F, int sf16, float *x, float *sx, const float *const *p, float *tmp) {
  const float *ln_w = p[0], *ln_b = p[1], *mk = p[2], *mr = p[3], *kw = p[4], *vw = p[5], *rw = p[6];
  float *xx = tmp, *kx = tmp + C, *rx = tmp + 2 * C, *r = tmp + 3 * C, *out = tmp + 4 * C,
        *kk = tmp + 5 * C;
  layernorm(x, ln_w, ln_b, C, xx);
  mix(xx, sx, mk, C, kx);
  mix(xx, sx, mr, C, rx);
  matvec(rx, rw, C, C, r);
  matvec(kx, kw, C, F, kk);
  for (int i = 0; i < F; ++i) { float t = kk[i] > 0.f ? kk[i] : 0.f; kk[i] = t * t; }
  matvec(kk, vw, F, C, out);
  for (int i = 0; i < C; ++i) { x[i] += sigmoidf_(r[i]) * out[i]; sx[i] = state_round(xx[i], sf16); }
}

/* ---------------------------------------------------------------- whole model */

size_t orc_state_floats(const orc_cfg *c) {
  if (c->version == 4) return (size_t)c->n_layer * 5 * c->n_embd;
  size_t S = c->n_embd / c->n_head;
  return (size_t)c->n_layer * (2 * (size_t)c->n_embd + (size_t)c->n_head * S * S);
}

/* Initial state, model.cpp:145-177: zeros, pp = -1e30. */
void orc_state_reset(const orc_cfg *c, float *state) {
  size_t n = orc_state_floats(c);
  memset(state, 0, n * sizeof(float));
  if (c->version == 4) {
    for (int l = 0; l < c->n_layer; ++l) {
      float *pp = state + ((size_t)l * 5 + 3) * c->n_embd;
      for (int i = 0; i < c->n_embd; ++i) pp[i] = -1e30f;
    }
  }
}

static int params_per_layer(int version) { return version == 4 ? 18 : version == 50 ? 20 : 22; }

/* One token through the model: kernels/default/model_forward.cpp:22-193 (embedding row
 * :87, layer loop :107-176 with the /2 at :173-175, ln_out + head :180-188).
 * params: fp32 arrays in the order kernels/default/init_model.cpp:75-126 pushes them.
 * state v4: [L][5][C] = sx, aa, bb, pp, ffn_sx (model.cpp:149-162);
 * state v5: per layer sx[C], s[H*S*S], ffn_sx[C] (model.cpp:163-175). */
int orc_forward(const orc_cfg *c, const float *const *params, const float *emb, float *state, int id,
                float *logits) {
  const int C = c->n_embd, F = c->n_ffn, L = c->n_layer, H = c->n_head;
  if (id < 0 || id >= c->vocab) return -1;
  float *x = (float *)malloc(sizeof(float) * C);
  float *tmp = (float *)malloc(sizeof(float) * ((size_t)10 * C + F));
  memcpy(x, emb + (size_t)id * C, sizeof(float) * C);
  const int ppl = params_per_layer(c->version), natt = ppl - 7;
  for (int l = 0; l < L; ++l) {
    const float *const *p = params + (size_t)l * ppl;
    if (c->version == 4) {
      float *st = state + (size_t)l * 5 * C;
      att_v4(C, c->state_fp16, x, st, st + C, st + 2 * C, st + 3 * C, p, tmp);
      ffn(C, F, c->state_fp16, x, st + 4 * C, p + natt, tmp);
    } else {
      size_t S = C / H, per = 2 * (size_t)C + (size_t)H * S * S;
      float *st = state + (size_t)l * per;
      att_v5(c->version, C, H, c->state_fp16, c->gate_from_xx, x, st, st + C, p, tmp);
      ffn(C, F, c->state_fp16, x, st + C + (size_t)H * S * S, p + natt, tmp);
    }
    if (c->rescale_every > 0 && (l + 1) % c->rescale_every == 0)
      for (int i = 0; i < C; ++i) x[i] *= 0.5f;
  }
  if (logits) {   /* a caller that walks a prompt only wants the last token's logits (model_forward_seq.cpp:170-179) */
    const float *const *p = params + (size_t)L * ppl;
    layernorm(x, p[0], p[1], C, tmp);
    matvec(tmp, p[2], C, c->vocab, logits);
  }
  free(x);
  free(tmp);
  return 0;
}

/* ---------------------------------------------------------------- quantisers */

/* fp32 -> fp16 bits, round to nearest even (IEEE binary16), and back. */
static uint16_t f32_to_f16(float f) {
  uint32_t x; memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
  if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);            /* overflow -> inf */
  if (x < 0x33000001u) return (uint16_t)sign;                          /* underflow -> 0 */
  int e = (int)(x >> 23) - 127;
  uint32_t m = (x & 0x7fffffu) | 0x800000u;
  int shift = e >= -14 ? 13 : 13 + (-14 - e);
  uint32_t half = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
  if (rem > mid || (rem == mid && (half & 1))) ++half;
  if (e >= -14) half += (uint32_t)(e + 14) << 10; /* mantissa carry bumps the exponent */
  return (uint16_t)(sign | half);
}

static float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31, m = h & 0x3ffu, x;
  if (e == 0) {
    if (m == 0) x = sign;
    else { int s = 0; while (!(m & 0x400u)) { m <<= 1; ++s; } x = sign | ((uint32_t)(113 - s) << 23) | ((m & 0x3ffu) << 13); }
  } else if (e == 31) x = sign | 0x7f800000u | (m << 13);
  else x = sign | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &x, 4);
  return f;
}

void orc_f32_to_f16(const float *src, uint16_t *dst, size_t n) { for (size_t i = 0; i < n; ++i) dst[i] = f32_to_f16(src[i]); }
void orc_f16_to_f32(const uint16_t *src, float *dst, size_t n) { for (size_t i = 0; i < n; ++i) dst[i] = f16_to_f32(src[i]); }

/* Round half away from zero, the behaviour of std::lround that the reference's own
 * quantisers use (kernels/export-ncnn/kernels.cpp:425,574,702).  x - trunc(x) is exact. */
static int round_half_away(float x) {
  float t = truncf(x);
  if (fabsf(x - t) >= 0.5f) t += x < 0.f ? -1.f : 1.f;
  return (int)t;
}

/* Scale of a block with absolute maximum amax mapped to qmax; 1 when the block is all
 * zero or the quotient underflows fp16 (cf. kernels/export-ncnn/kernels.cpp:389-393). */
static uint16_t block_scale(float amax, float qmax) {
  uint16_t s = f32_to_f16(amax / qmax);
  if ((s & 0x7fffu) == 0 || (s & 0x7c00u) == 0x7c00u) s = 0x3c00u;
  return s;
}

/* int8: symmetric, one fp16 scale per OUTPUT channel n = fp16(max_k |W[k,n]| / 127),
 * q = clamp(round(W / scale), -127, 127).  W is [K,N] (in,out); q is [N][K]. */
void orc_quant_int8(const float *W, int K, int N, int8_t *q, uint16_t *scales) {
  for (int n = 0; n < N; ++n) {
    float amax = 0.f;
    for (int k = 0; k < K; ++k) { float a = fabsf(W[(size_t)k * N + n]); if (a > amax) amax = a; }
    uint16_t sh = block_scale(amax, 127.f);
    float s = f16_to_f32(sh);
    scales[n] = sh;
    for (int k = 0; k < K; ++k) {
      int v = round_half_away(W[(size_t)k * N + n] / s);
      v = v > 127 ? 127 : v < -127 ? -127 : v;
      q[(size_t)n * K + k] = (int8_t)v;
    }
  }
}

/* int4: symmetric, groups of 32 consecutive INPUT indices per output channel,
 * scale = fp16(max|W| / 7), q in [-7,7] stored as the nibble q + 8, two per byte with
 * the even k in the low nibble.  packed is [N][K/2], scales [N][K/32]. */
void orc_quant_int4(const float *W, int K, int N, uint8_t *packed, uint16_t *scales) {
  const int G = K / 32;
  for (int n = 0; n < N; ++n)
    for (int g = 0; g < G; ++g) {
      float amax = 0.f;
      for (int k = g * 32; k < g * 32 + 32; ++k) { float a = fabsf(W[(size_t)k * N + n]); if (a > amax) amax = a; }
      uint16_t sh = block_scale(amax, 7.f);
      float s = f16_to_f32(sh);
      scales[(size_t)n * G + g] = sh;
      for (int k = g * 32; k < g * 32 + 32; k += 2) {
        int v0 = round_half_away(W[(size_t)k * N + n] / s), v1 = round_half_away(W[(size_t)(k + 1) * N + n] / s);
        v0 = v0 > 7 ? 7 : v0 < -7 ? -7 : v0;
        v1 = v1 > 7 ? 7 : v1 < -7 ? -7 : v1;
        packed[(size_t)n * (K / 2) + k / 2] = (uint8_t)((v0 + 8) | ((v1 + 8) << 4));
      }
    }
}

/* Dequantise back to a [K,N] fp32 matrix: float(q) * float(scale), exact in fp32. */
void orc_dequant_int8(const int8_t *q, const uint16_t *scales, int K, int N, float *W) {
  for (int n = 0; n < N; ++n) {
    float s = f16_to_f32(scales[n]);
    for (int k = 0; k < K; ++k) W[(size_t)k * N + n] = (float)q[(size_t)n * K + k] * s;
  }
}

void orc_dequant_int4(const uint8_t *packed, const uint16_t *scales, int K, int N, float *W) {
  const int G = K / 32;
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      uint8_t b = packed[(size_t)n * (K / 2) + k / 2];
      int qv = (int)((k & 1) ? (b >> 4) : (b & 15)) - 8;
      W[(size_t)k * N + n] = (float)qv * f16_to_f32(scales[(size_t)n * G + k / 32]);
    }
}
