// Where the [64 steps][64 features] blocks of the sequence tensors lie, and how they are fetched.
//
// Every sequence tensor of a call is a 2-D array of 16-bit elements, rows = batch item x time,
// described to the copy engine by a tensor map (cuTensorMapEncodeTiled); a chunk's block of one
// tensor is ONE tiled bulk copy (cp.async.bulk.tensor.2d) of a 64 x 64 box that lands as a dense
// row-major [64][64] block in shared memory.  The plain operators pass [B*T, 64] arrays; the fused
// layer entry points pass the projection output [B*T, 4*H*64] (query | key | value | gate, heads
// inside a row) and read the heads in place, so no folded copies of the tensors are ever made.
// Rows of a box that fall outside the array arrive as zeros; rows that belong to the next batch
// item (a partial last chunk) are overwritten with identity steps by the kernels.
#pragma once

#include <cuda.h>

#include "async_copy.cuh"
#include "common.cuh"

namespace t2fw {
namespace seq {

constexpr int kMaxTensors = 6;

enum : int {
  kUnitForget = 1,     // the d-side gate is the constant 1: nothing is read for it
  kSigmoidGate = 2,    // the k-side gate tensor holds pre-activations: gate = max(sigmoid(g), 1/8)
  kContiguous = 4,     // every tensor is a dense [rows][64] array: a chunk's block is one linear 8 KB copy
  kOutByRow = 8,       // outputs are [problem row][T][64] arrays (one per sub-item), not windows of a batch item's row
};
constexpr float kGateFloor = 0.125f;   // with gates >= 1/8 no 32-step product leaves the safe range

struct Maps {
  CUtensorMap m[kMaxTensors];    // one per input tensor of the kernel
  const void *base[kMaxTensors]; // the arrays themselves (used for the linear copies of dense [rows][64] arrays)
  int col[kMaxTensors];          // column of sub-item 0 in a row of that tensor (elements)
  int hdiv[kMaxTensors];         // sub-item h of a batch item reads the 64-column window number
  int hmod[kMaxTensors];         //   (h / hdiv) % hmod of that tensor
  int heads;                     // sub-items per batch item: problem row bh = b * heads + h.  Heads of a
                                 // layer: hdiv = 1, hmod = heads.  A D x K state cut into 64 x 64 blocks:
                                 // h = i * (K/64) + j, d-side tensors hdiv = K/64, hmod = D/64, k-side 1, K/64
  int flags;
  float q_scale;                 // factor on the query tensor (1 for the plain operators)
};

// an output tensor: element (row of the 2-D array, feature) at p[row * ld + col + 64 * h + feature]
template <typename T>
struct Out {
  T *p;
  int64_t ld;
  int col;
};

// box (64 features x 64 rows) with its first row `row` and first column `col` -> dst (8 KB, 128-byte aligned)
__device__ __forceinline__ void load_block(void *dst, const CUtensorMap *map, int col, int row, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          acp::smem_u32(dst)),
      "l"(map), "r"(col), "r"(row), "r"(acp::smem_u32(bar))
      : "memory");
}

// ---- in-place transforms of a raw [64][64] block in shared memory (all threads of the CTA) ------
template <typename T>
__device__ __forceinline__ void fill_block(T *blk, float v, int tid, int nthreads) {
  const T tv = (T)v;
  for (int i = tid; i < 64 * 64; i += nthreads) blk[i] = tv;
}
// gate = max(sigmoid(g), 1/8), rounded to the storage type (what a separate elementwise pass
// followed by the plain operator would have fed the kernel)
template <typename T>
__device__ __forceinline__ void sigmoid_gate_block(T *blk, int tid, int nthreads) {
  for (int i = tid; i < 64 * 64; i += nthreads) {
    const float g = Elem<T>::ld(blk + i);
    blk[i] = (T)fmaxf(__fdividef(1.f, 1.f + __expf(-g)), kGateFloor);
  }
}
template <typename T>
__device__ __forceinline__ void scale_block(T *blk, float s, int tid, int nthreads) {
  for (int i = tid; i < 64 * 64; i += nthreads) blk[i] = (T)(Elem<T>::ld(blk + i) * s);
}

// The block of tensor i for the chunk whose first row is `row` (nv valid rows), sub-item h.
// Dense [rows][64] arrays: one linear bulk copy of the valid rows; otherwise the tiled copy of the
// whole box.  Returns the bytes that will arrive on the barrier.
template <typename T>
__device__ __forceinline__ uint32_t fetch_block(const Maps &mp, int i, void *dst, int row, int h, int nv, uint64_t *bar) {
  if (mp.flags & kContiguous) {
    const uint32_t bytes = (uint32_t)nv * 64u * sizeof(T);
    acp::bulk_g2s(dst, static_cast<const T *>(mp.base[i]) + (size_t)row * 64, bytes, bar);
    return bytes;
  }
  load_block(dst, &mp.m[i], mp.col[i] + ((h / mp.hdiv[i]) % mp.hmod[i]) * 64, row, bar);
  return 64u * 64u * sizeof(T);
}

// host: tensor map of a [rows][cols] array of 16-bit elements with `ld` elements between rows
int make_map(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t ld);

}  // namespace seq
}  // namespace t2fw
