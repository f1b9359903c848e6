// fr_b200_matvec_noalloc: the streaming dequant-matvec for callers that must not allocate.
//
// Some hosts hand a plugin a fixed memory budget and forbid any further allocation once they are running: an
// inference server whose execute callback may not call cudaMalloc because the call serialises the whole device
// and can fail when the framework's own pool already owns the memory, or a real-time loop that has to keep its
// latency bounded.  fr_b200_matvec needs scratch beyond its inputs and outputs (the fp16 / quantised copy of the
// matrix, the packed streaming tiles, row scales, a padded output and the phase descriptor) and takes it from
// cudaMalloc on every call.  This variant keeps that scratch in a fixed array inside the library image instead.
//
// The array lives in every GPU context that loads the library, until the process exits.  All calls share it and it
// keeps what the last call left: everything that must start from zero is cleared here, and two calls whose GPU
// work overlaps (different streams, different threads) race on it — callers serialise.
// In host code the array's name is only a handle for the runtime, not a device address; the address is looked up
// with cudaGetSymbolAddress once per device, with that device current, the first time the entry point runs on
// it.  Make that first call outside any stream capture.
#include <atomic>
#include <cstring>
#include <string>

#include "../../include/fr_b200.h"
#include "internal.h"

using namespace frb;

namespace {

constexpr size_t MAX_WEIGHTS = 1u << 20;          // padded rows x K
constexpr int MAX_ROWS = 16384, MAX_K = 8192;
constexpr size_t OFF_STAGE = 0;                   // fp16 copy, or int8 / int4 canonical codes      (<= 2 MiB)
constexpr size_t OFF_SCALES = 2u << 20;           // canonical scales                               (<= 128 KiB)
constexpr size_t OFF_TILES = OFF_SCALES + (128u << 10);   // packed streaming tiles                  (<= 2 MiB)
constexpr size_t OFF_RSCALE = OFF_TILES + (2u << 20);     // int8 row scales of the padded rows      (<= 32 KiB)
constexpr size_t OFF_Y = OFF_RSCALE + (32u << 10);        // [8][padded rows] fp32 + status word     (<= 512 KiB + 256)
constexpr size_t OFF_PHASE = OFF_Y + (512u << 10) + 256;  // PhaseDev
constexpr size_t SCRATCH_BYTES = OFF_PHASE + 256;

static __device__ __align__(256) unsigned char g_scratch[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
// device address of g_scratch on each device, once looked up.  The address belongs to the device's primary context:
// after a cudaDeviceReset the entry point must not be used again in this process.
std::atomic<unsigned char *> g_scratch_addr[MAX_DEVICES];

thread_local std::string g_noalloc_err;

}  // namespace

extern "C" const char *fr_b200_noalloc_last_error(void) { return g_noalloc_err.c_str(); }

#define NA_FAIL(code, msg) do { g_noalloc_err = (msg); return (code); } while (0)
#define NA_CU(call)                                                                          \
  do {                                                                                       \
    cudaError_t e_ = (call);                                                                 \
    if (e_ != cudaSuccess) NA_FAIL(FR_B200_E_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)); \
  } while (0)

extern "C" int fr_b200_matvec_noalloc(const float *W, int K, int N, int weight_format, const float *x, int batch,
                                      float *y, int device, void *stream) {
  if (!W || !x || !y) NA_FAIL(FR_B200_E_ARG, "null pointer");
  if (K <= 0 || N <= 0 || K % 64) NA_FAIL(FR_B200_E_ARG, "K must be a positive multiple of 64");
  if (weight_format < 0 || weight_format > 2) NA_FAIL(FR_B200_E_ARG, "bad weight_format");
  if (batch < 1 || batch > MAX_B) NA_FAIL(FR_B200_E_ARG, "batch must be 1..8");
  if (device < 0 || device >= MAX_DEVICES) NA_FAIL(FR_B200_E_ARG, "device ordinal out of range");
  // the kernel reads x with 16-byte loads straight from the caller's buffer (fr_b200_matvec copies it first)
  if (reinterpret_cast<uintptr_t>(x) & 15) NA_FAIL(FR_B200_E_ARG, "x must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(W) & 3) || (reinterpret_cast<uintptr_t>(y) & 3)) NA_FAIL(FR_B200_E_ARG, "W and y must be 4-byte aligned");
  const int Npad = (N + ROWS - 1) / ROWS * ROWS, nb = Npad / ROWS;
  if (K > MAX_K || Npad > MAX_ROWS || (size_t)Npad * K > MAX_WEIGHTS)
    NA_FAIL(FR_B200_E_UNSUPPORTED, "matrix exceeds the built-in scratch: at most 1,048,576 weights after padding the "
                                   "rows to a multiple of 16, K <= 8192, N <= 16384");
  NA_CU(cudaSetDevice(device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  {
    // the call copies a status word back and synchronises the stream: neither is legal while the stream is capturing
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    NA_CU(cudaStreamIsCapturing(st, &cap));
    if (cap != cudaStreamCaptureStatusNone) NA_FAIL(FR_B200_E_STATE, "the stream is capturing: this entry point synchronises it");
  }
  unsigned char *S = g_scratch_addr[device].load(std::memory_order_acquire);
  if (!S) {
    // first call on this device: resolve the device address of the array (the host-side name is not one)
    unsigned char *ptr = nullptr;
    NA_CU(cudaGetSymbolAddress((void **)&ptr, g_scratch));
    g_scratch_addr[device].store(ptr, std::memory_order_release);
    S = ptr;
  }
  const int fmt = weight_format;
  const size_t n = (size_t)K * N, rb = rowblock_bytes(fmt, K);
  uint8_t *tiles = S + OFF_TILES;
  __half *rscale = reinterpret_cast<__half *>(S + OFF_RSCALE);
  float *ypad = reinterpret_cast<float *>(S + OFF_Y);
  int *status = reinterpret_cast<int *>(ypad + (size_t)batch * Npad);
  PhaseDev *phd = reinterpret_cast<PhaseDev *>(S + OFF_PHASE);

  // the array keeps the previous call's contents: clear what this call reads before writing
  NA_CU(cudaMemsetAsync(rscale, 0, (size_t)Npad * 2, st));
  NA_CU(cudaMemsetAsync(ypad, 0, ((size_t)batch * Npad + 1) * 4, st));
  if (fmt == FMT_FP16) {
    __half *w16 = reinterpret_cast<__half *>(S + OFF_STAGE);
    NA_CU(launch_f32_to_f16(W, w16, n, st));
    NA_CU(launch_pack(fmt, w16, nullptr, K, N, tiles, rb, nullptr, 0, st));
  } else if (fmt == FMT_INT8) {
    int8_t *q = reinterpret_cast<int8_t *>(S + OFF_STAGE);
    __half *sc = reinterpret_cast<__half *>(S + OFF_SCALES);
    NA_CU(launch_quant_int8(W, K, N, q, sc, st));
    NA_CU(launch_pack(fmt, q, sc, K, N, tiles, rb, rscale, ROWS, st));
  } else {
    uint8_t *q = S + OFF_STAGE;
    __half *sc = reinterpret_cast<__half *>(S + OFF_SCALES);
    NA_CU(launch_quant_int4(W, K, N, q, sc, st));
    NA_CU(launch_pack(fmt, q, sc, K, N, tiles, rb, nullptr, 0, st));
  }
  PhaseDev ph;
  std::memset(&ph, 0, sizeof(ph));
  ph.w = tiles; ph.rscale = rscale; ph.kind = PH_MATVEC; ph.K = K; ph.n_items = nb; ph.n_sub = 1;
  NA_CU(cudaMemcpyAsync(phd, &ph, sizeof(ph), cudaMemcpyHostToDevice, st));   // pageable source: staged by the driver before return
  DecodeParams p;
  std::memset(&p, 0, sizeof(p));
  // C only sizes the operand space, max(3*C, F) * batch halfs
  p.version = 4; p.L = 0; p.C = 64; p.F = K; p.V = N; p.Vpad = Npad; p.fmt = fmt; p.B = batch; p.n_phases = 1;
  p.phases = phd; p.kk = reinterpret_cast<exch_t *>(const_cast<float *>(x)); p.logits = ypad; p.status = status;
  const int mode = decode_mode(batch);
  int optin = 0, grid = 0, stages = 0;
  NA_CU(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  for (int s = 6; s >= 2; --s)
    if (decode_smem_bytes(fmt, mode, 64, K, 4, s) <= (size_t)optin) { stages = s; break; }
  if (!stages) NA_FAIL(FR_B200_E_UNSUPPORTED, "K too large for shared memory at this batch size");
  p.n_stages = stages;
  const size_t smem = decode_smem_bytes(fmt, mode, 64, K, 4, stages);
  NA_CU(decode_max_grid(fmt, mode, smem, device, &grid));
  if (!grid) NA_FAIL(FR_B200_E_UNSUPPORTED, "kernel does not fit on an SM");
  NA_CU(launch_decode(p, mode, grid, smem, st));
  NA_CU(cudaMemcpy2DAsync(y, (size_t)N * 4, ypad, (size_t)Npad * 4, (size_t)N * 4, batch, cudaMemcpyDeviceToDevice, st));
  int hstatus = 0;
  NA_CU(cudaMemcpyAsync(&hstatus, status, 4, cudaMemcpyDeviceToHost, st));
  NA_CU(cudaStreamSynchronize(st));
  if (hstatus) NA_FAIL(FR_B200_E_TIMEOUT, "device-side wait timed out (code " + std::to_string(hstatus) + ")");
  return FR_B200_OK;
}
