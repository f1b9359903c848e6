// Streaming tile layout of the projection matrices, shared by host code and kernels.
//
// A matrix with N outputs and K inputs is cut into row blocks of 16 outputs.  A row block is
// streamed as stages of at most kt_max(fmt) input positions; a stage is one contiguous piece of
// HBM (one TMA bulk copy).  Inside a stage the data sits in the order the tensor-core fragments of
// mma.m16n8k16 consume it, so a warp reads its operands with conflict-free 128-bit shared loads:
//
//   chunk  = 64 consecutive inputs k (4 MMAs j = 0..3 of 16 inputs each)
//   lane   = 4*g + q  (g = 0..7 picks rows g and g+8 of the block, q = 0..3 picks 4 inputs of the 16)
//   lane's inputs of MMA j: k0 = 64*chunk + 16*j + 4*q, elements k0..k0+3
//
//   fp16  chunk = [j][lane][16 B]           16 B = W[g][k0,k0+1] W[g+8][k0,k0+1] W[g][k0+2,k0+3] W[g+8][k0+2,k0+3]
//   int8  chunk = [j/2][lane][16 B]         8 B per j, same element order, one byte each, stored as q + 128
//   int4  chunk = [lane][16 B]              4 B per j: nibble i (bits 4i..4i+3) holds, for i = 0..7,
//                                           W[g][k0] W[g+8][k0] W[g][k0+2] W[g+8][k0+2] W[g][k0+1] W[g+8][k0+1] W[g][k0+3] W[g+8][k0+3]
//                                           each stored as q + 8
//   int4 stage = all chunk weights, then per chunk 64 B of fp16 group scales [g][grp0 row g, grp0 row g+8,
//                grp1 row g, grp1 row g+8] (group = 32 inputs = MMAs {0,1} / {2,3} of the chunk)
//   int8 row scales live in a separate fp16 array, one per output row.
#pragma once
#include <stdint.h>

#ifdef __CUDACC__
#define FRB_HD __host__ __device__ __forceinline__
#else
#define FRB_HD inline
#endif

namespace frb {

constexpr int FMT_FP16 = 0, FMT_INT8 = 1, FMT_INT4 = 2;
constexpr int ROWS = 16;      // outputs per row block
constexpr int CHUNK_K = 64;   // inputs per chunk

FRB_HD int kt_max(int fmt) { return fmt == FMT_FP16 ? 1024 : 2048; }   // inputs per stage
FRB_HD int chunk_weight_bytes(int fmt) { return fmt == FMT_FP16 ? 2048 : fmt == FMT_INT8 ? 1024 : 512; }
FRB_HD int chunk_bytes(int fmt) { return chunk_weight_bytes(fmt) + (fmt == FMT_INT4 ? 64 : 0); }
// bytes of a stage covering kt inputs (kt a multiple of 64)
FRB_HD uint32_t stage_bytes(int fmt, int kt) { return (uint32_t)(kt / CHUNK_K) * (uint32_t)chunk_bytes(fmt); }
FRB_HD int num_stages(int fmt, int K) { return (K + kt_max(fmt) - 1) / kt_max(fmt); }
// bytes of one row block over all K inputs
FRB_HD uint32_t rowblock_bytes(int fmt, int K) { return (uint32_t)(K / CHUNK_K) * (uint32_t)chunk_bytes(fmt); }
// bytes of one ring slot = the largest stage of the format (fp16 / int8: 32 KiB, int4: 18 KiB)
FRB_HD uint32_t slot_bytes(int fmt) { return (uint32_t)(kt_max(fmt) / CHUNK_K) * (uint32_t)chunk_bytes(fmt); }

// Element position of input k, batch column n inside the fp16 operand vector a CTA keeps in shared
// memory (NB = padded batch, 1 or 8): [chunk][j/2][n][q][(j&1)*4 + s] with k = 64*chunk + 16*j + 4*q + s.
FRB_HD int xs_index(int k, int n, int NB) {
  int c = k >> 6, j = (k >> 4) & 3, q = (k >> 2) & 3, s = k & 3;
  return ((((c * 2 + (j >> 1)) * NB + n) * 4 + q) << 3) + ((j & 1) << 2) + s;
}

}  // namespace frb
