// Building blocks of the chunked decay-rule kernels (D = K = 64, 16-bit storage).
//
// A chunk is 64 time steps = 4 sub-blocks of 16.  Inside a sub-block the decay is factored with
// cumulative gate products (inclusive prefixes gp[t] = g_first..g_t per column):
//     Qt = q * gp        Kt = k / gp        (k side, gates f_key)
//     dOt = dO * ap      Xt = x / ap        (d side, gates f)
// so that for i <= t inside the block  Qt_t . Kt_i = sum_k q_t k_i prod_{i<j<=t} g_j.  Only
// products over at most 16 steps are ever inverted, and only one-sided (fp32/TF32 range).
// Across sub-blocks everything is anchored division-free: prefixes for (Qt, dOt), and
// "to-the-end-of-block" factors Kt * gI, Xt * aI (gI, aI = whole-block products) for the
// operands that enter the state / state-gradient updates.  All contractions run on tensor cores
// as TF32 m16n8k8 MMAs with fp32 accumulation; the D x K state stays in fp32 accumulators.
#pragma once

#include "common.cuh"

namespace t2fw {
namespace chunk {

constexpr int kC = 64;         // chunk length = checkpoint interval
constexpr int kSub = 16;       // sub-block length
constexpr int kNSub = kC / kSub;
constexpr int kDim = 64;       // D = K = 64
constexpr int kLd = 68;        // row stride (floats) of the 64-wide operand tiles
constexpr int kLdP = 20;       // row stride of the 16x16 pair tiles
constexpr int kThreads = 128;
constexpr float kTiny = 9.094947e-13f;      // 2^-40: smallest gate magnitude used in products
constexpr float kRangeLo = 7.888609e-31f;   // 2^-100
constexpr float kRangeHi = 1.267651e+30f;   // 2^100

__device__ __forceinline__ uint32_t to_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float round_tf32(float v) { return __uint_as_float(to_tf32(v)); }

// D[16x8] += A[16x8] * B[8x8], TF32 operands, fp32 accumulate.
// Fragment layout (g = lane >> 2, tq = lane & 3):
//   a0 = A[g][tq], a1 = A[g+8][tq], a2 = A[g][tq+4], a3 = A[g+8][tq+4]
//   b0 = B[tq][g], b1 = B[tq+4][g]
//   c0 = C[g][2tq], c1 = C[g][2tq+1], c2 = C[g+8][2tq], c3 = C[g+8][2tq+1]
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Fragment loaders from row-major fp32 tiles holding TF32-rounded values.
//   lda  : A[m][k] = t[(m0+m)*ld + k0+k]        lda_t: A[m][k] = t[(k0+k)*ld + m0+m]
//   ldb  : B[k][n] = t[(k0+k)*ld + n0+n]        ldb_t: B[k][n] = t[(n0+n)*ld + k0+k]
__device__ __forceinline__ void lda(uint32_t (&a)[4], const float *t, int ld, int m0, int k0, int g, int tq) {
  a[0] = __float_as_uint(t[(m0 + g) * ld + k0 + tq]);
  a[1] = __float_as_uint(t[(m0 + g + 8) * ld + k0 + tq]);
  a[2] = __float_as_uint(t[(m0 + g) * ld + k0 + tq + 4]);
  a[3] = __float_as_uint(t[(m0 + g + 8) * ld + k0 + tq + 4]);
}
__device__ __forceinline__ void lda_t(uint32_t (&a)[4], const float *t, int ld, int m0, int k0, int g, int tq) {
  a[0] = __float_as_uint(t[(k0 + tq) * ld + m0 + g]);
  a[1] = __float_as_uint(t[(k0 + tq) * ld + m0 + g + 8]);
  a[2] = __float_as_uint(t[(k0 + tq + 4) * ld + m0 + g]);
  a[3] = __float_as_uint(t[(k0 + tq + 4) * ld + m0 + g + 8]);
}
__device__ __forceinline__ void ldb(uint32_t (&b)[2], const float *t, int ld, int k0, int n0, int g, int tq) {
  b[0] = __float_as_uint(t[(k0 + tq) * ld + n0 + g]);
  b[1] = __float_as_uint(t[(k0 + tq + 4) * ld + n0 + g]);
}
__device__ __forceinline__ void ldb_t(uint32_t (&b)[2], const float *t, int ld, int k0, int n0, int g, int tq) {
  b[0] = __float_as_uint(t[(n0 + g) * ld + k0 + tq]);
  b[1] = __float_as_uint(t[(n0 + g) * ld + k0 + tq + 4]);
}
// Same as lda_t / ldb but every element is multiplied by a per-column (lda_t: per-m, ldb: per-n)
// factor first: used for the "to the end of the block" operands Xt*aI and Kt*gI.
__device__ __forceinline__ void lda_t_scaled(uint32_t (&a)[4], const float *t, int ld, int m0, int k0,
                                             int g, int tq, float s_lo, float s_hi) {
  a[0] = to_tf32(t[(k0 + tq) * ld + m0 + g] * s_lo);
  a[1] = to_tf32(t[(k0 + tq) * ld + m0 + g + 8] * s_hi);
  a[2] = to_tf32(t[(k0 + tq + 4) * ld + m0 + g] * s_lo);
  a[3] = to_tf32(t[(k0 + tq + 4) * ld + m0 + g + 8] * s_hi);
}
__device__ __forceinline__ void ldb_scaled(uint32_t (&b)[2], const float *t, int ld, int k0, int n0,
                                           int g, int tq, float s) {
  b[0] = to_tf32(t[(k0 + tq) * ld + n0 + g] * s);
  b[1] = to_tf32(t[(k0 + tq + 4) * ld + n0 + g] * s);
}

template <typename T> struct Pair;
template <> struct Pair<__half> {
  static __device__ __forceinline__ float2 ld(const __half *p) {
    return __half22float2(*reinterpret_cast<const __half2 *>(p));
  }
  static __device__ __forceinline__ void st(__half *p, float a, float b) {
    *reinterpret_cast<__half2 *>(p) = __floats2half2_rn(a, b);
  }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 ld(const __nv_bfloat16 *p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
  }
  static __device__ __forceinline__ void st(__nv_bfloat16 *p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(a, b);
  }
};

__device__ __forceinline__ float sanitize_gate(float g) {
  return fabsf(g) < kTiny ? copysignf(kTiny, g) : g;
}

// One side (k side or d side) of the operand preparation for one chunk.
//   gate, mul, div : global pointers to row 0 of the chunk for this batch row ([rows][64]),
//                    mul / div may be null
//   out_mul[row][c] = tf32(mul * prefix)     out_div[row][c] = tf32(div / prefix)
//   out_pre[row][c] = prefix (fp32)          out_raw[row][c] = sanitized gate (fp32)
//   blk[I][c]       = product of the gates of sub-block I
// Warp I handles sub-block I; lane l handles columns 2l, 2l+1.  Rows >= nvalid are identity
// steps (gate 1, zero vectors).  Returns true if a prefix left [2^-100, 2^100] or is not finite.
template <typename T>
__device__ __forceinline__ bool prep_side(const T *__restrict__ gate, const T *__restrict__ mul,
                                          const T *__restrict__ div, int nvalid, float *out_mul,
                                          float *out_div, float *out_pre, float *out_raw, float *blk,
                                          int tid = -1) {
  if (tid < 0) tid = threadIdx.x;       // callers with more than 128 threads pass a 0..127 index
  const int I = tid >> 5;
  const int c = (tid & 31) * 2;
  float2 gv[kSub], mv[kSub], dv[kSub];
#pragma unroll
  for (int t = 0; t < kSub; ++t) {
    const int row = I * kSub + t;
    const bool in = row < nvalid;
    gv[t] = in ? Pair<T>::ld(gate + (size_t)row * kDim + c) : make_float2(1.f, 1.f);
    mv[t] = (in && mul) ? Pair<T>::ld(mul + (size_t)row * kDim + c) : make_float2(0.f, 0.f);
    dv[t] = (in && div) ? Pair<T>::ld(div + (size_t)row * kDim + c) : make_float2(0.f, 0.f);
  }
  float p0 = 1.f, p1 = 1.f, lo = 1.f, hi = 1.f;
#pragma unroll
  for (int t = 0; t < kSub; ++t) {
    const int row = I * kSub + t;
    const float g0 = sanitize_gate(gv[t].x), g1 = sanitize_gate(gv[t].y);
    p0 *= g0;
    p1 *= g1;
    lo = fminf(lo, fminf(fabsf(p0), fabsf(p1)));
    hi = fmaxf(hi, fmaxf(fabsf(p0), fabsf(p1)));
    if (out_mul) {
      *reinterpret_cast<float2 *>(out_mul + row * kLd + c) =
          make_float2(round_tf32(mv[t].x * p0), round_tf32(mv[t].y * p1));
    }
    if (out_div) {
      *reinterpret_cast<float2 *>(out_div + row * kLd + c) =
          make_float2(round_tf32(__fdividef(dv[t].x, p0)), round_tf32(__fdividef(dv[t].y, p1)));
    }
    if (out_pre) *reinterpret_cast<float2 *>(out_pre + row * kLd + c) = make_float2(p0, p1);
    if (out_raw) *reinterpret_cast<float2 *>(out_raw + row * kLd + c) = make_float2(g0, g1);
  }
  *reinterpret_cast<float2 *>(blk + I * kDim + c) = make_float2(p0, p1);
  // !(x >= lo) also catches NaN
  return !(lo >= kRangeLo) || !(hi <= kRangeHi);
}

// ---- pieces shared by the backward kernels --------------------------------------------------
// A[m][k] = t[(m0+m)*ld + k0+k] * sc[k0+k]  (per-contraction-index scale)
__device__ __forceinline__ void lda_colscaled(uint32_t (&a)[4], const float *t, int ld, int m0, int k0,
                                              int g, int tq, const float *sc) {
  const float s0 = sc[k0 + tq], s1 = sc[k0 + tq + 4];
  a[0] = to_tf32(t[(m0 + g) * ld + k0 + tq] * s0);
  a[1] = to_tf32(t[(m0 + g + 8) * ld + k0 + tq] * s0);
  a[2] = to_tf32(t[(m0 + g) * ld + k0 + tq + 4] * s1);
  a[3] = to_tf32(t[(m0 + g + 8) * ld + k0 + tq + 4] * s1);
}

// state step on accumulator registers (warp w owns rows 16w..16w+15, all 64 columns):
//   S <- (aI gI^T) .* S + (Xt aI)^T (Kt gI)   for sub-block I
__device__ __forceinline__ void state_step_regs(float (&S)[8][4], const float *Xt, const float *Kt,
                                                const float *aI, const float *gI, int I, int w, int g,
                                                int tq) {
  const float a_lo = aI[I * kDim + 16 * w + g], a_hi = aI[I * kDim + 16 * w + g + 8];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const float2 gg = *reinterpret_cast<const float2 *>(gI + I * kDim + nt * 8 + 2 * tq);
    S[nt][0] *= a_lo * gg.x;
    S[nt][1] *= a_lo * gg.y;
    S[nt][2] *= a_hi * gg.x;
    S[nt][3] *= a_hi * gg.y;
  }
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    uint32_t a[4];
    lda_t_scaled(a, Xt, kLd, 16 * w, I * kSub + 8 * ks, g, tq, a_lo, a_hi);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      uint32_t b[2];
      ldb_scaled(b, Kt, kLd, I * kSub + 8 * ks, nt * 8, g, tq, gI[I * kDim + nt * 8 + g]);
      mma_tf32(S[nt], a, b);
    }
  }
}

// state-gradient step: R <- (aI gI^T) .* R + dOt_I^T Qt_I
__device__ __forceinline__ void grad_step_regs(float (&R)[8][4], const float *dOt, const float *Qt,
                                               const float *aI, const float *gI, int I, int w, int g,
                                               int tq, bool scale_old) {
  if (scale_old) {
    const float a_lo = aI[I * kDim + 16 * w + g], a_hi = aI[I * kDim + 16 * w + g + 8];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float2 gg = *reinterpret_cast<const float2 *>(gI + I * kDim + nt * 8 + 2 * tq);
      R[nt][0] *= a_lo * gg.x;
      R[nt][1] *= a_lo * gg.y;
      R[nt][2] *= a_hi * gg.x;
      R[nt][3] *= a_hi * gg.y;
    }
  }
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    uint32_t a[4];
    lda_t(a, dOt, kLd, 16 * w, I * kSub + 8 * ks, g, tq);   // A[d][s] = dOt[s][d]
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      uint32_t b[2];
      ldb(b, Qt, kLd, I * kSub + 8 * ks, nt * 8, g, tq);    // B[s][k] = Qt[s][k]
      mma_tf32(R[nt], a, b);
    }
  }
}

// inclusive suffix / exclusive prefix sums over the 16 rows of a sub-block for values held in
// the MMA accumulator layout (row g -> lo, row g+8 -> hi; lanes with equal tq share a column)
__device__ __forceinline__ void suffix16(float &lo, float &hi, int g, int tq) {
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    const float yl = __shfl_down_sync(0xffffffffu, lo, 4 * o);
    const float yh = __shfl_down_sync(0xffffffffu, hi, 4 * o);
    if (g + o < 8) { lo += yl; hi += yh; }
  }
  lo += __shfl_sync(0xffffffffu, hi, tq);   // g = 0 holds the whole upper half
}
__device__ __forceinline__ void exclusive_prefix16(float &lo, float &hi, int g, int tq) {
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    const float yl = __shfl_up_sync(0xffffffffu, lo, 4 * o);
    const float yh = __shfl_up_sync(0xffffffffu, hi, 4 * o);
    if (g >= o) { lo += yl; hi += yh; }
  }
  const float tot_lo = __shfl_sync(0xffffffffu, lo, 28 + tq);  // g = 7 holds the whole lower half
  const float el = __shfl_up_sync(0xffffffffu, lo, 4);
  const float eh = __shfl_up_sync(0xffffffffu, hi, 4);
  lo = (g >= 1) ? el : 0.f;
  hi = ((g >= 1) ? eh : 0.f) + tot_lo;
}

}  // namespace chunk
}  // namespace t2fw
