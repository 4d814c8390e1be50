// Building blocks of the 64-step chunk kernels of the decay rule (D = K = 64, 16-bit storage):
// lfw_c64_fwd.cu (outputs of a chunk) and lfw_c64_bwd.cu (the five sequence gradients).
//
// Algebra.  A chunk is 64 steps t = 0..63 with gates a_t (d side, `forget`) and g_t (k side,
// `f_key`).  With cumulative products A_t = a_0..a_t, G_t = g_0..g_t and the anchor REF = 31 in
// the middle of the chunk, the in-chunk decay between two steps factors into ratios to the anchor
//     pm_g[t] = G_t / G_REF        (t > REF: product of g_{REF+1..t};  t <= REF: 1 / product of g_{t+1..REF})
// so that no product over more than 32 steps is ever formed or inverted, and only one-sided.
// "mid" operands carry these ratios (q * pm_g, k / pm_g, dO * pm_a, x / pm_a); their pair products
// P = tril((q pm_g)(k / pm_g)^T), Z = tril((dO pm_a)(x / pm_a)^T) are the exact in-chunk decays.
// Terms that involve the state at the chunk start use operands anchored at the chunk START
// (q * G_t, dO * A_t) and terms that involve the state gradient at the chunk end use operands
// anchored at the chunk END (k * G_63/G_s, x * A_63/A_s): those products only ever decay, so an
// underflow there loses nothing that the exact result would keep.  The 64 x 64 state blocks are
// scaled on ONE side only (by the anchor products of the side whose gradients are formed).
// A batch row whose one-sided 32-step products leave [2^-100, 2^100] is flagged and recomputed by
// the sequential scan kernels.
//
// Operand tiles are 64 x 64 fp32 (TF32-rounded) in the K-major 128-byte-swizzle layout of the
// tcgen05 shared-memory descriptor: two column blocks of 32 floats; inside a block row r is 128
// bytes at r * 128 and its eight 16-byte chunks are XOR-ed with (r % 8).  A tile [rows][cols] is
// the A or B operand of a product that contracts over `cols`.  Every wait is bounded.
#pragma once

#include "async_copy.cuh"
#include "common.cuh"
#include "umma.cuh"

namespace t2fw {
namespace c64 {

constexpr int kC = 64;                 // chunk length = checkpoint interval
constexpr int kDim = 64;               // D = K = 64
constexpr int kRef = 31;               // anchor: after step 31
constexpr int kTile = 64 * 64 * 4;     // bytes of one operand tile
constexpr int kColBlock = 64 * 128;    // bytes of one 32-column block of a tile
constexpr int kRawBytes = kC * kDim * 2;
constexpr float kTinyState = 9.094947e-13f;     // 2^-40: smallest gate magnitude used in products
constexpr float kTinyGate = 9.765625e-4f;       // 2^-10: below this the exact gate-gradient formula is used
constexpr float kRangeLo = 7.888609e-31f;       // 2^-100
constexpr float kRangeHi = 1.267651e+30f;       // 2^100

// byte offset of element (r, c) of a tile
__device__ __forceinline__ int toff(int r, int c) {
  return (c >> 5) * kColBlock + r * 128 + ((((c >> 2) & 7) ^ (r & 7)) << 4) + ((c & 3) << 2);
}

__device__ __forceinline__ float rna_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

__device__ __forceinline__ float sanitize_gate(float g) {
  return fabsf(g) < kTinyState ? copysignf(kTinyState, g) : g;
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// D[64 x 32] (+)= A[64 x 64] * B[rows n0 .. n0+31][64]^T over the 64 contraction columns (8 steps of 8)
__device__ __forceinline__ void mma_64x32x64(uint32_t d_tmem, uint32_t a_tile, uint32_t b_tile, int n0,
                                             bool accumulate) {
  constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t o = (uint32_t)((ks >> 2) * kColBlock + (ks & 3) * 32);
    umma::mma_tf32(d_tmem, desc_sw128(a_tile + o), desc_sw128(b_tile + (uint32_t)n0 * 128u + o), idesc,
                   accumulate || ks > 0);
  }
}
// both 32-column halves of a 64 x 64 result: columns 0-31 into lanes 0-15 of every lane quarter,
// columns 32-63 into lanes 16-31, both at tensor-memory column `col`
__device__ __forceinline__ void mma_64x64x64(uint32_t tmem_base, int col, uint32_t a_tile, uint32_t b_tile,
                                             bool accumulate) {
  mma_64x32x64(umma::tmem_addr(tmem_base, 0, col), a_tile, b_tile, 0, accumulate);
  mma_64x32x64(umma::tmem_addr(tmem_base, 16, col), a_tile, b_tile, 32, accumulate);
}

__device__ __forceinline__ void sync_all() {
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
}

// Gate products of one feature over one 16-step quarter of a chunk.
//   g[j]   : sanitized gates of steps 16*tq + j (1 beyond the valid steps)
//   returns the product of the quarter
template <typename T>
__device__ __forceinline__ float load_gates16(const T *gate_col, int tq, int nvalid, float (&g)[16]) {
  float p = 1.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int t = 16 * tq + j;
    g[j] = sanitize_gate(t < nvalid ? Elem<T>::ld(gate_col + t * kDim) : 1.f);
    p *= g[j];
  }
  return p;
}

// Walks the 16 steps of quarter tq of one feature in the order in which the ratio to the anchor
// is a running product (downwards from the anchor for tq < 2, upwards for tq >= 2) and calls
//   fn(j, t, mulfac, divfac)      mulfac = pm[t] = G_t / G_REF,  divfac = 1 / pm[t]
// with j the compile-time index into g[] (t = 16 * tq + j).  `carry` is the product of the
// quarter between this one and the anchor (1 for the two inner quarters).
// Returns false if a running product left [2^-100, 2^100] (or is not finite).
template <typename F>
__device__ __forceinline__ bool walk_quarter(int tq, const float (&g)[16], float carry, F &&fn) {
  float s = carry, lo = fabsf(carry), hi = lo;
  if (tq < 2) {
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) {
      const int j = 15 - jj;
      fn(j, 16 * tq + j, __fdividef(1.f, s), s);     // s = product of the gates after t, up to the anchor
      s *= g[j];
      lo = fminf(lo, fabsf(s));
      hi = fmaxf(hi, fabsf(s));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      s *= g[j];
      lo = fminf(lo, fabsf(s));
      hi = fmaxf(hi, fabsf(s));
      fn(j, 16 * tq + j, s, __fdividef(1.f, s));
    }
  }
  return (lo >= kRangeLo) && (hi <= kRangeHi);     // false for NaN as well
}

}  // namespace c64
}  // namespace t2fw
