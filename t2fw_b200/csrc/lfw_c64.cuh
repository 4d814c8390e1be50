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
// Below this gate magnitude the pair terms of the gate gradient are summed directly.  The factored
// form divides a cancelled sum by the gate; measured against the step-by-step result its error is
// 7e-4 of the largest gradient for gates of 2^-13, 3e-3 at 2^-14.5, 5e-3 at 2^-16.5 and 4e-2 at
// 2^-18.5 (tolerance 2e-2).  Every entry costs a chunk of the pass a few hundred cycles, and N(0,1)
// gates fall below 2^-10 three times per chunk, below 2^-13 0.4 times.
constexpr float kTinyGate = 1.220703125e-4f;    // 2^-13
constexpr float kRangeLo = 7.888609e-31f;       // 2^-100
constexpr float kRangeHi = 1.267651e+30f;       // 2^100

// byte offset of element (r, c) of a tile
__device__ __forceinline__ int toff(int r, int c) {
  return (c >> 5) * kColBlock + r * 128 + ((((c >> 2) & 7) ^ (r & 7)) << 4) + ((c & 3) << 2);
}

// Round to TF32 (10 mantissa bits), nearest with ties away from zero - what cvt.rna.tf32.f32 does -
// as two integer instructions: the conversion instruction runs on the quarter-rate pipe and there
// are hundreds of them per thread and chunk.  (Infinity becomes NaN; such rows are flagged anyway.)
__device__ __forceinline__ float rna_tf32(float v) {
  return __uint_as_float((__float_as_uint(v) + 0x1000u) & 0xffffe000u);
}

// The same rounding for a value that is ONLY stored as a tensor-core operand: the tensor core ignores
// the low 13 bits of an fp32 operand (shared memory and tensor memory alike; tests/test_umma_gpu.py checks it),
// so adding half a unit of the last kept place is enough and the mask can be left out.
__device__ __forceinline__ float bias_tf32(float v) { return __uint_as_float(__float_as_uint(v) + 0x1000u); }

__device__ __forceinline__ float sanitize_gate(float g) {
  return fabsf(g) < kTinyState ? copysignf(kTinyState, g) : g;
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// D[64 x 32] (+)= A[64 x 64] * B[rows n0 .. n0+31][64]^T over the 64 contraction columns (8 steps of 8).
// da, db are the descriptors of the two tiles (desc_sw128 of the tile base); a k-step or a row
// offset only moves the start-address field, which is the low word in units of 16 bytes.
__device__ __forceinline__ void mma_64x32x64(uint32_t d_tmem, uint64_t da, uint64_t db, int n0, bool accumulate) {
  constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
  const uint64_t dbn = db + (uint64_t)(n0 * 128 >> 4);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
    umma::mma_tf32(d_tmem, da + o, dbn + o, idesc, accumulate || ks > 0);
  }
}

// D[tmem] (+)= A[tmem] * B[smem]^T: the A operand is read from tensor memory (row r of an M = 64
// operand in lane 32 * (r / 16) + r % 16 of a lane set, one 32-bit column per contraction index).
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t desc_b, uint32_t idesc,
                                            bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u, zero = 0u;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(desc_b), "r"(idesc), "r"(acc), "r"(zero)
      : "memory");
}

// D[64 x 32] (+)= A * B[rows n0 .. n0+31][64]^T with the 64 x 64 A operand in tensor memory (64 columns
// starting at a_tmem, whose lane field selects the lane set that also receives D)
__device__ __forceinline__ void mma_ts_64x32x64(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, int n0,
                                                bool accumulate) {
  constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
  const uint64_t dbn = db + (uint64_t)(n0 * 128 >> 4);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
    mma_tf32_ts(d_tmem, a_tmem + 8 * ks, dbn + o, idesc, accumulate || ks > 0);
  }
}

__device__ __forceinline__ void tmem_st8(uint32_t addr, const float (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"r"(addr),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
               "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
               "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
               : "memory");
}

// An A operand row block in tensor memory, stored twice.  The tensor core reads row r of A from
// the lane in which it produces row r of D, and the two 32-column halves of every result live in
// the two lane sets (lanes 0-15 / 16-31 of a lane quarter), so both lane sets need all 64 columns
// of A.  Lane fl of the lower half warp holds columns 8 * part .. + 7 of row 16 * q4 + fl, lane
// fl + 16 holds columns 32 + 8 * part .. + 7 of the same row; a tcgen05.st names ONE column range
// for the whole warp, so the halves swap their values by shuffle and store twice.
__device__ __forceinline__ void tmem_put_dup(uint32_t lane_base_col, int part, int h, const float (&v)[8]) {
  float lo[8], hi[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float p = __shfl_xor_sync(0xffffffffu, v[j], 16);
    lo[j] = h ? p : v[j];
    hi[j] = h ? v[j] : p;
  }
  tmem_st8(lane_base_col + 8 * part, lo);
  tmem_st8(lane_base_col + 32 + 8 * part, hi);
}

// 16-byte asynchronous copy global -> shared (no register, no scoreboard)
__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(umma::smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// One lane of a converged warp.  The MMA-issuing code runs with the whole warp converged on
// warp-uniform values (so the descriptors live in uniform registers) and only the instruction
// itself is predicated on the elected lane.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
// warp index as a value the compiler knows to be the same in all lanes
__device__ __forceinline__ int uniform_warp_idx() { return __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0); }

// Work item -> (problem row, chunk) and problem row -> (batch item, head) with 32-bit divisions
// (the launchers refuse problems with 2^31 or more chunks or rows).
struct Item {
  int bh, c, b, h;
};
__device__ __forceinline__ Item split_item(int64_t ci, int64_t nc, int heads) {
  Item it;
  const uint32_t u = (uint32_t)ci, n = (uint32_t)nc;
  it.bh = (int)(u / n);
  it.c = (int)(u - (uint32_t)it.bh * n);
  it.b = (int)((uint32_t)it.bh / (uint32_t)heads);
  it.h = it.bh - it.b * heads;
  return it;
}

__device__ __forceinline__ void sync_all() {
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
}

// ---- operand preparation, stage 1: ratios to the anchor ------------------------------------
// Thread (feature, 16-step quarter tq).  g[j] = sanitized gate of step 16 * tq + j (the raw gate
// blocks hold 1 beyond the valid steps); returns the product of the quarter.
template <typename T>
__device__ __forceinline__ float load_gates16(const T *gate_col, int tq, float (&g)[16], float *min_abs = nullptr) {
  float mn = kRangeHi;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    g[j] = Elem<T>::ld(gate_col + (16 * tq + j) * kDim);
    mn = fminf(mn, fabsf(g[j]));
  }
  if (!(mn >= kTinyState)) {      // rare (also NaN): some gate needs the clamp
#pragma unroll
    for (int j = 0; j < 16; ++j) g[j] = sanitize_gate(g[j]);
  }
  float p = 1.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) p *= g[j];
  if (min_abs != nullptr) *min_abs = mn;
  return p;
}

// pm[j] = G_t / G_REF for t = 16 * tq + j: a running product downwards from the anchor for
// tq < 2 (then inverted), upwards for tq >= 2.  `carry` is the product of the quarter between this
// one and the anchor (1 for the two inner quarters).  Returns false if a running product left
// [2^-100, 2^100] or is not finite.
__device__ __forceinline__ bool ratios16(int tq, const float (&g)[16], float carry, float (&pm)[16]) {
  float s = carry, lo = fabsf(carry), hi = lo;
  if (tq < 2) {
#pragma unroll
    for (int j = 15; j >= 0; --j) {
      pm[j] = __fdividef(1.f, s);     // s = product of the gates after t, up to the anchor
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
      pm[j] = s;
    }
  }
  return (lo >= kRangeLo) && (hi <= kRangeHi);     // false for NaN as well
}

// ---- stage 2: scaled operand tiles ------------------------------------------------------------
template <typename T> struct Vec4;     // four consecutive 16-bit values -> four floats
template <> struct Vec4<__half> {
  static __device__ __forceinline__ float4 ld(const __half *p) {
    const uint2 u = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld(const __nv_bfloat16 *p) {
    const uint2 u = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
};
template <typename T> struct Vec2;     // two consecutive 16-bit values -> two floats
template <> struct Vec2<__half> {
  static __device__ __forceinline__ float2 ld(const __half *p) {
    return __half22float2(*reinterpret_cast<const __half2 *>(p));
  }
};
template <> struct Vec2<__nv_bfloat16> {
  static __device__ __forceinline__ float2 ld(const __nv_bfloat16 *p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
  }
};
__device__ __forceinline__ float4 bias4(float4 v) {
  return make_float4(bias_tf32(v.x), bias_tf32(v.y), bias_tf32(v.z), bias_tf32(v.w));
}
__device__ __forceinline__ float4 mul4(float4 a, float4 b) {
  return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w);
}
__device__ __forceinline__ float4 rcp4(float4 a) {
  return make_float4(__fdividef(1.f, a.x), __fdividef(1.f, a.y), __fdividef(1.f, a.z), __fdividef(1.f, a.w));
}

// A partial chunk (nvalid < 64): the steps beyond the valid ones become identity steps.  The raw
// blocks are [nblk][64][64]; block i is a gate block if bit i of gate_mask is set.
template <typename T>
__device__ __forceinline__ void pad_raw_tail(T *raw, int nblk, unsigned gate_mask, int nvalid, int tid,
                                             int nthreads) {
  const int per = (kC - nvalid) * kDim;
  for (int i = tid; i < nblk * per; i += nthreads) {
    const int blk = i / per, o = i % per;
    raw[blk * kC * kDim + nvalid * kDim + o] = (T)(((gate_mask >> blk) & 1u) ? 1.f : 0.f);
  }
}

}  // namespace c64
}  // namespace t2fw
