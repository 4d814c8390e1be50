// Chunked decay-rule backward for D = K = 64, 16-bit storage (algebra in lfw_chunk.cuh).
//
// Replaces the reference's reverse scan, five einsums and two in-place multiplies
// (t2fw/csrc/lfw_kernel.cu:61-102, t2fw/csrc/lfw.cpp:84-93) with three launches:
//   1. lfw_chunk_bwd_local_kernel  (b, chunk): the chunk's own contribution G_c to the state
//      gradient at the chunk start, and the chunk's decay vectors
//   2. lfw_chunk_bwd_carry_kernel  reverse elementwise scan over chunks: state gradient at the
//      END of every chunk (fp32, in place over G_c) and d_state
//   3. lfw_chunk_bwd_main_kernel   (b, chunk): the four sub-blocks in reverse; the forward state
//      is recomputed from the chunk's checkpoint, the state gradient R is carried in fp32
//      accumulators, and d_x, d_f, d_q, d_k, d_f_key come out of TF32 MMAs plus fp32 scans.
//
// Per sub-block (start state S0, end gradient R, block decays aI, gI, prefixes ap, gp):
//   dq = gp .* (dOt S0 + Z Kt)                     Z = tril(dOt Xt^T)
//   dk = (Z^T Qt + gI .* (Xt aI) R) ./ gp           P = tril(Qt Kt^T)
//   dx = (P^T dOt + aI .* (Kt gI) R^T) ./ ap
//   R_prev = (aI gI^T) .* R + dOt^T Qt
// Gate gradients use the scaling identity restarted at every sub-block end,
//   g_t dg_t = sum_{s>=t}(q_s dq_s - k_s dk_s) + sum_d (R .* S)_end ,
// evaluated term by term so that only the in-block pair terms cancel, and those are built
// from identical TF32-rounded operands on both sides:
//   H = suffix_t[ Qt.*(dOt S0 + Z Kt) - Kt.*(Z^T Qt) ] + exclusive_prefix_t[ Kt.*gI.*((Xt aI) R) ]
//       + gI .* sum_d aI R S0 ;   d_f_key = H / g        (d side: same with the roles exchanged)
#include <type_traits>

#include "lfw_chunk.cuh"

namespace t2fw {

using namespace chunk;

namespace {

struct BwdScratch {
  float *G, *Ac, *Gc;
  int *flags, *rowflag;
};

inline size_t bwd_scratch_floats(int64_t B, int64_t nc) {
  return (size_t)B * nc * kDim * kDim + 2 * (size_t)B * nc * kDim + (size_t)B * nc + (size_t)B;
}

inline BwdScratch carve(void *scratch, int64_t B, int64_t nc) {
  BwdScratch s;
  s.G = static_cast<float *>(scratch);
  s.Ac = s.G + (size_t)B * nc * kDim * kDim;
  s.Gc = s.Ac + (size_t)B * nc * kDim;
  s.flags = reinterpret_cast<int *>(s.Gc + (size_t)B * nc * kDim);
  s.rowflag = s.flags + (size_t)B * nc;
  return s;
}

// A[m][k] = t[(m0+m)*ld + k0+k] * sc[k0+k]  (per-contraction-index scale)
__device__ __forceinline__ void lda_colscaled(uint32_t (&a)[4], const float *t, int ld, int m0, int k0,
                                              int g, int tq, const float *sc) {
  const float s0 = sc[k0 + tq], s1 = sc[k0 + tq + 4];
  a[0] = to_tf32(t[(m0 + g) * ld + k0 + tq] * s0);
  a[1] = to_tf32(t[(m0 + g + 8) * ld + k0 + tq] * s0);
  a[2] = to_tf32(t[(m0 + g) * ld + k0 + tq + 4] * s1);
  a[3] = to_tf32(t[(m0 + g + 8) * ld + k0 + tq + 4] * s1);
}

// forward state step (same as in the forward file): S <- (aI gI^T).*S + (Xt aI)^T (Kt gI)
__device__ __forceinline__ void state_step(float (&S)[8][4], const float *Xt, const float *Kt,
                                           const float *aI, const float *gI, int I, int w, int g, int tq) {
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

// state-gradient step: R <- (aI gI^T).*R + dOt_I^T Qt_I
__device__ __forceinline__ void grad_step(float (&R)[8][4], const float *dOt, const float *Qt,
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

template <typename T>
__global__ void __launch_bounds__(kThreads)
lfw_chunk_bwd_local_kernel(const T *__restrict__ go, const T *__restrict__ f, const T *__restrict__ q,
                           const T *__restrict__ fk, float *__restrict__ G, float *__restrict__ Ac,
                           float *__restrict__ Gc, int *__restrict__ flags, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *dOt = sm, *Qt = dOt + kC * kLd, *aI = Qt + kC * kLd, *gI = aI + kNSub * kDim;
  __shared__ int s_flag;
  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc;
  const int64_t t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  if (threadIdx.x == 0) s_flag = 0;
  __syncthreads();
  const size_t base = ((size_t)b * T_ + t0) * kDim;
  bool bad = prep_side<T>(fk + base, q + base, nullptr, nvalid, Qt, nullptr, nullptr, nullptr, gI);
  bad |= prep_side<T>(f + base, go + base, nullptr, nvalid, dOt, nullptr, nullptr, nullptr, aI);
  if (bad) s_flag = 1;
  __syncthreads();

  float R[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) R[nt][0] = R[nt][1] = R[nt][2] = R[nt][3] = 0.f;
#pragma unroll
  for (int I = kNSub - 1; I >= 0; --I) grad_step(R, dOt, Qt, aI, gI, I, w, g, tq, I < kNSub - 1);

  float *Gp_ = G + ((size_t)b * nc + c) * kDim * kDim;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<float2 *>(Gp_ + (16 * w + g) * kDim + nt * 8 + 2 * tq) = make_float2(R[nt][0], R[nt][1]);
    *reinterpret_cast<float2 *>(Gp_ + (16 * w + g + 8) * kDim + nt * 8 + 2 * tq) = make_float2(R[nt][2], R[nt][3]);
  }
  if (threadIdx.x < kDim) {
    const int d = threadIdx.x;
    Ac[((size_t)b * nc + c) * kDim + d] = aI[d] * aI[kDim + d] * aI[2 * kDim + d] * aI[3 * kDim + d];
  } else {
    const int kk = threadIdx.x - kDim;
    Gc[((size_t)b * nc + c) * kDim + kk] = gI[kk] * gI[kDim + kk] * gI[2 * kDim + kk] * gI[3 * kDim + kk];
  }
  if (threadIdx.x == 0) flags[(size_t)b * nc + c] = s_flag;
}

// R_end(c-1) = (Ac Gc^T) R_end(c) + G_c, from the last chunk (R_end = grad_state) down; G_c is
// overwritten with R_end(c).  The value left after chunk 0 is d_state.
template <typename T>
__global__ void __launch_bounds__(128)
lfw_chunk_bwd_carry_kernel(const T *__restrict__ grad_state, float *__restrict__ G,
                           const float *__restrict__ Ac, const float *__restrict__ Gc,
                           const int *__restrict__ flags, int *__restrict__ rowflag,
                           T *__restrict__ d_state, int64_t B, int64_t nc) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * kDim * (kDim / 4)) return;
  const int64_t b = idx / (kDim * (kDim / 4));
  const int d = (int)((idx / (kDim / 4)) % kDim);
  const int k0 = (int)(idx % (kDim / 4)) * 4;
  const T *sp = grad_state + ((size_t)b * kDim + d) * kDim + k0;
  float2 s01 = Pair<T>::ld(sp), s23 = Pair<T>::ld(sp + 2);
  float R[4] = {s01.x, s01.y, s23.x, s23.y};
  int any = 0;
  // batches of 8 chunks, last chunk first: loads of a batch precede its dependent FMA chain
  for (int64_t c0 = nc - 1; c0 >= 0; c0 -= 8) {
    float4 l[8], gg[8];
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t c = (c0 - j >= 0) ? c0 - j : 0;
      const size_t bc = (size_t)b * nc + c;
      l[j] = *reinterpret_cast<const float4 *>(G + (bc * kDim + d) * kDim + k0);
      a[j] = Ac[bc * kDim + d];
      gg[j] = *reinterpret_cast<const float4 *>(Gc + bc * kDim + k0);
      if (d == 0 && k0 == 0) any |= flags[bc];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (c0 - j >= 0) {
        const size_t bc = (size_t)b * nc + c0 - j;
        *reinterpret_cast<float4 *>(G + (bc * kDim + d) * kDim + k0) = make_float4(R[0], R[1], R[2], R[3]);
        R[0] = a[j] * gg[j].x * R[0] + l[j].x;
        R[1] = a[j] * gg[j].y * R[1] + l[j].y;
        R[2] = a[j] * gg[j].z * R[2] + l[j].z;
        R[3] = a[j] * gg[j].w * R[3] + l[j].w;
      }
    }
  }
  T *dp = d_state + ((size_t)b * kDim + d) * kDim + k0;
  Pair<T>::st(dp, R[0], R[1]);
  Pair<T>::st(dp + 2, R[2], R[3]);
  if (d == 0 && k0 == 0) rowflag[b] = any;
}

// inclusive suffix / exclusive prefix sums over the 16 rows of a sub-block for values held in
// the MMA accumulator layout (row g -> v_lo, row g+8 -> v_hi; lanes with equal tq share a column)
__device__ __forceinline__ void suffix16(float &lo, float &hi, int g, int tq) {
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    const float yl = __shfl_down_sync(0xffffffffu, lo, 4 * o);
    const float yh = __shfl_down_sync(0xffffffffu, hi, 4 * o);
    if (g + o < 8) { lo += yl; hi += yh; }
  }
  const float tot_hi = __shfl_sync(0xffffffffu, hi, tq);   // g = 0 holds the whole upper half
  lo += tot_hi;
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

constexpr int kStgLd = kDim + 8;   // row stride (elements) of the 16-bit output staging tiles
constexpr int kFixCap = 256;       // tiny-gate elements per sub-block that get the exact formula
constexpr float kTinyGate = 9.765625e-4f;   // 2^-10: below this |gate| the cancelling form is not used

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
lfw_chunk_bwd_main_kernel(const T *__restrict__ go, const T *__restrict__ x, const T *__restrict__ f,
                          const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ fk,
                          const T *__restrict__ state, const T *__restrict__ ckpt,
                          const float *__restrict__ Rend, T *__restrict__ dx, T *__restrict__ df,
                          T *__restrict__ dq, T *__restrict__ dk, T *__restrict__ dfk,
                          int *__restrict__ rowflag, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Qt = sm, *Kt = Qt + kC * kLd, *Xt = Kt + kC * kLd, *dOt = Xt + kC * kLd;
  float *Gp = dOt + kC * kLd, *Ap = Gp + kC * kLd;
  float *S0 = Ap + kC * kLd, *Rm = S0 + kDim * kLd;
  float *Pr = Rm + kDim * kLd, *Zr = Pr + kNSub * kSub * kLdP;
  float *aI = Zr + kNSub * kSub * kLdP, *gI = aI + kNSub * kDim;
  float *colpart = gI + kNSub * kDim;           // [4][64] partial column sums of R.*S0
  float *c4d = colpart + 4 * kDim;              // [64]
  int *fix_list = reinterpret_cast<int *>(c4d + kDim);        // [kFixCap] tiny-gate elements
  T *stg = reinterpret_cast<T *>(fix_list + kFixCap);         // 5 tiles [16][kStgLd]
  __shared__ int fix_n;

  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc;
  const int64_t t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const size_t base = ((size_t)b * T_ + t0) * kDim;
  prep_side<T>(fk + base, q + base, k + base, nvalid, Qt, Kt, Gp, nullptr, gI);
  prep_side<T>(f + base, go + base, x + base, nvalid, dOt, Xt, Ap, nullptr, aI);
  __syncthreads();

  // pair tiles of sub-block w: P = tril(Qt Kt^T), Z = tril(dOt Xt^T)
  {
    float accP[2][4] = {}, accZ[2][4] = {};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t a[4], a2[4];
      lda(a, Qt, kLd, 16 * w, 8 * ks, g, tq);
      lda(a2, dOt, kLd, 16 * w, 8 * ks, g, tq);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        uint32_t bb[2], b2[2];
        ldb_t(bb, Kt, kLd, 8 * ks, 16 * w + 8 * nt, g, tq);
        ldb_t(b2, Xt, kLd, 8 * ks, 16 * w + 8 * nt, g, tq);
        mma_tf32(accP[nt], a, bb);
        mma_tf32(accZ[nt], a2, b2);
      }
    }
    float *Pw = Pr + w * kSub * kLdP, *Zw = Zr + w * kSub * kLdP;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int i0 = 8 * nt + 2 * tq;
      Pw[g * kLdP + i0] = (i0 <= g) ? round_tf32(accP[nt][0]) : 0.f;
      Pw[g * kLdP + i0 + 1] = (i0 + 1 <= g) ? round_tf32(accP[nt][1]) : 0.f;
      Pw[(g + 8) * kLdP + i0] = (i0 <= g + 8) ? round_tf32(accP[nt][2]) : 0.f;
      Pw[(g + 8) * kLdP + i0 + 1] = (i0 + 1 <= g + 8) ? round_tf32(accP[nt][3]) : 0.f;
      Zw[g * kLdP + i0] = (i0 <= g) ? round_tf32(accZ[nt][0]) : 0.f;
      Zw[g * kLdP + i0 + 1] = (i0 + 1 <= g) ? round_tf32(accZ[nt][1]) : 0.f;
      Zw[(g + 8) * kLdP + i0] = (i0 <= g + 8) ? round_tf32(accZ[nt][2]) : 0.f;
      Zw[(g + 8) * kLdP + i0 + 1] = (i0 + 1 <= g + 8) ? round_tf32(accZ[nt][3]) : 0.f;
    }
  }

  // state gradient at the end of the chunk: rows 16w+g / +8, columns nt*8 + 2tq, +1
  float R[8][4];
  {
    const float *Rc = Rend + ((size_t)b * nc + c) * kDim * kDim;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float2 lo = *reinterpret_cast<const float2 *>(Rc + (16 * w + g) * kDim + nt * 8 + 2 * tq);
      const float2 hi = *reinterpret_cast<const float2 *>(Rc + (16 * w + g + 8) * kDim + nt * 8 + 2 * tq);
      R[nt][0] = lo.x; R[nt][1] = lo.y; R[nt][2] = hi.x; R[nt][3] = hi.y;
    }
  }
  const T *Sc = (c == 0) ? state + (size_t)b * kDim * kDim
                         : ckpt + ((size_t)b * nc + (c - 1)) * kDim * kDim;

#pragma unroll 1
  for (int I = kNSub - 1; I >= 0; --I) {
    if (threadIdx.x == 0) fix_n = 0;
    // ---- state at the start of sub-block I, recomputed from the chunk's checkpoint ----------
    {
      float S[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float2 lo = Pair<T>::ld(Sc + (16 * w + g) * kDim + nt * 8 + 2 * tq);
        const float2 hi = Pair<T>::ld(Sc + (16 * w + g + 8) * kDim + nt * 8 + 2 * tq);
        S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
      }
#pragma unroll 1
      for (int J = 0; J < I; ++J) state_step(S, Xt, Kt, aI, gI, J, w, g, tq);

      // boundary terms sum(R.*S0) with the block decay, then publish S0 and R for the MMAs
      const float a_lo = aI[I * kDim + 16 * w + g], a_hi = aI[I * kDim + 16 * w + g + 8];
      float row_lo = 0.f, row_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float2 gg = *reinterpret_cast<const float2 *>(gI + I * kDim + nt * 8 + 2 * tq);
        const float p0 = R[nt][0] * S[nt][0], p1 = R[nt][1] * S[nt][1];
        const float p2 = R[nt][2] * S[nt][2], p3 = R[nt][3] * S[nt][3];
        row_lo += gg.x * p0 + gg.y * p1;
        row_hi += gg.x * p2 + gg.y * p3;
        float c0 = a_lo * p0 + a_hi * p2, c1 = a_lo * p1 + a_hi * p3;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          c0 += __shfl_xor_sync(0xffffffffu, c0, o);
          c1 += __shfl_xor_sync(0xffffffffu, c1, o);
        }
        if (g == 0) {
          colpart[w * kDim + nt * 8 + 2 * tq] = c0;
          colpart[w * kDim + nt * 8 + 2 * tq + 1] = c1;
        }
        *reinterpret_cast<float2 *>(S0 + (16 * w + g) * kLd + nt * 8 + 2 * tq) =
            make_float2(round_tf32(S[nt][0]), round_tf32(S[nt][1]));
        *reinterpret_cast<float2 *>(S0 + (16 * w + g + 8) * kLd + nt * 8 + 2 * tq) =
            make_float2(round_tf32(S[nt][2]), round_tf32(S[nt][3]));
        *reinterpret_cast<float2 *>(Rm + (16 * w + g) * kLd + nt * 8 + 2 * tq) =
            make_float2(round_tf32(R[nt][0]), round_tf32(R[nt][1]));
        *reinterpret_cast<float2 *>(Rm + (16 * w + g + 8) * kLd + nt * 8 + 2 * tq) =
            make_float2(round_tf32(R[nt][2]), round_tf32(R[nt][3]));
      }
      row_lo += __shfl_xor_sync(0xffffffffu, row_lo, 1);
      row_lo += __shfl_xor_sync(0xffffffffu, row_lo, 2);
      row_hi += __shfl_xor_sync(0xffffffffu, row_hi, 1);
      row_hi += __shfl_xor_sync(0xffffffffu, row_hi, 2);
      if (tq == 0) {
        c4d[16 * w + g] = a_lo * row_lo;
        c4d[16 * w + g + 8] = a_hi * row_hi;
      }
    }
    __syncthreads();

    const float *PI = Pr + I * kSub * kLdP, *ZI = Zr + I * kSub * kLdP;
    const float *aIb = aI + I * kDim, *gIb = gI + I * kDim;
    const int r0 = I * kSub;          // first row of the sub-block inside the chunk
    const int n0 = 16 * w;            // this warp's 16-column slice (k side and d side)

    // ================= k side: d_q, d_k, d_f_key for columns n0..n0+15 =====================
    {
      float TQ[2][4] = {}, T2[2][4] = {}, T7[2][4] = {};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {       // contraction over d
        uint32_t a[4], a7[4];
        lda(a, dOt, kLd, r0, 8 * ks, g, tq);
        lda_colscaled(a7, Xt, kLd, r0, 8 * ks, g, tq, aIb);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          uint32_t bs[2], br[2];
          ldb(bs, S0, kLd, 8 * ks, n0 + 8 * nt, g, tq);
          ldb(br, Rm, kLd, 8 * ks, n0 + 8 * nt, g, tq);
          mma_tf32(TQ[nt], a, bs);
          mma_tf32(T7[nt], a7, br);
        }
      }
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {       // contraction over the 16 steps of the block
        uint32_t az[4], azt[4];
        lda(az, ZI, kLdP, 0, 8 * ks, g, tq);        // A[s][i] = Z[s][i]
        lda_t(azt, ZI, kLdP, 0, 8 * ks, g, tq);     // A[i][s] = Z[s][i]
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          uint32_t bk[2], bq[2];
          ldb(bk, Kt, kLd, r0 + 8 * ks, n0 + 8 * nt, g, tq);
          ldb(bq, Qt, kLd, r0 + 8 * ks, n0 + 8 * nt, g, tq);
          mma_tf32(TQ[nt], az, bk);
          mma_tf32(T2[nt], azt, bq);
        }
      }
      T *s_dq = stg, *s_dk = stg + kSub * kStgLd, *s_dfk = stg + 2 * kSub * kStgLd;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {          // the two adjacent columns
          const int col = n0 + 8 * nt + 2 * tq + e;
          const float gIk = gIb[col], c4 = gIk * (colpart[col] + colpart[kDim + col] +
                                                   colpart[2 * kDim + col] + colpart[3 * kDim + col]);
          float v[2], b3[2], rg[2], gprev[2], dqv[2], dkv[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {        // rows g and g+8
            const int row = r0 + g + 8 * h;
            const float tqv = TQ[nt][2 * h + e], t2 = T2[nt][2 * h + e], t7 = T7[nt][2 * h + e];
            const float qt = Qt[row * kLd + col], kt = Kt[row * kLd + col], gp = Gp[row * kLd + col];
            rg[h] = __fdividef(1.f, gp);
            gprev[h] = (g + 8 * h > 0) ? Gp[(row - 1) * kLd + col] : 1.f;
            dqv[h] = gp * tqv;
            dkv[h] = (t2 + gIk * t7) * rg[h];
            v[h] = qt * tqv - kt * t2;
            b3[h] = kt * gIk * t7;
          }
          suffix16(v[0], v[1], g, tq);
          exclusive_prefix16(b3[0], b3[1], g, tq);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float H = v[h] + b3[h] + c4;
            const int lr = g + 8 * h;
            s_dq[lr * kStgLd + col] = (T)dqv[h];
            s_dk[lr * kStgLd + col] = (T)dkv[h];
            s_dfk[lr * kStgLd + col] = (T)(H * gprev[h] * rg[h]);
            if (fabsf(gprev[h]) * kTinyGate > fabsf(Gp[(r0 + lr) * kLd + col])) {   // |g_t| < 2^-10
              const int slot = atomicAdd(&fix_n, 1);
              if (slot < kFixCap) fix_list[slot] = (lr << 8) | col;
            }
          }
        }
      }
    }
    // ================= d side: d_x, d_f for columns n0..n0+15 ===============================
    {
      float TO[2][4] = {}, T4[2][4] = {}, T8[2][4] = {};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {       // contraction over k
        uint32_t a[4], a8[4];
        lda(a, Qt, kLd, r0, 8 * ks, g, tq);
        lda_colscaled(a8, Kt, kLd, r0, 8 * ks, g, tq, gIb);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          uint32_t bs[2], br[2];
          ldb_t(bs, S0, kLd, 8 * ks, n0 + 8 * nt, g, tq);    // B[k][d] = S0[d][k]
          ldb_t(br, Rm, kLd, 8 * ks, n0 + 8 * nt, g, tq);    // B[k][d] = R[d][k]
          mma_tf32(TO[nt], a, bs);
          mma_tf32(T8[nt], a8, br);
        }
      }
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        uint32_t ap_[4], apt[4];
        lda(ap_, PI, kLdP, 0, 8 * ks, g, tq);       // A[t][i] = P[t][i]
        lda_t(apt, PI, kLdP, 0, 8 * ks, g, tq);     // A[i][t] = P[t][i]
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          uint32_t bx[2], bo[2];
          ldb(bx, Xt, kLd, r0 + 8 * ks, n0 + 8 * nt, g, tq);
          ldb(bo, dOt, kLd, r0 + 8 * ks, n0 + 8 * nt, g, tq);
          mma_tf32(TO[nt], ap_, bx);
          mma_tf32(T4[nt], apt, bo);
        }
      }
      T *s_dx = stg + 3 * kSub * kStgLd, *s_df = stg + 4 * kSub * kStgLd;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = n0 + 8 * nt + 2 * tq + e;
          const float aId = aIb[col], c4 = c4d[col];
          float v[2], b3[2], ra[2], aprev[2], dxv[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int row = r0 + g + 8 * h;
            const float to = TO[nt][2 * h + e], t4 = T4[nt][2 * h + e], t8 = T8[nt][2 * h + e];
            const float dot = dOt[row * kLd + col], xt = Xt[row * kLd + col], ap = Ap[row * kLd + col];
            ra[h] = __fdividef(1.f, ap);
            aprev[h] = (g + 8 * h > 0) ? Ap[(row - 1) * kLd + col] : 1.f;
            dxv[h] = (t4 + aId * t8) * ra[h];
            v[h] = dot * to - xt * t4;
            b3[h] = xt * aId * t8;
          }
          suffix16(v[0], v[1], g, tq);
          exclusive_prefix16(b3[0], b3[1], g, tq);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float H = v[h] + b3[h] + c4;
            const int lr = g + 8 * h;
            s_dx[lr * kStgLd + col] = (T)dxv[h];
            s_df[lr * kStgLd + col] = (T)(H * aprev[h] * ra[h]);
            if (fabsf(aprev[h]) * kTinyGate > fabsf(Ap[(r0 + lr) * kLd + col])) {   // |f_t| < 2^-10
              const int slot = atomicAdd(&fix_n, 1);
              if (slot < kFixCap) fix_list[slot] = (1 << 16) | (lr << 8) | col;
            }
          }
        }
      }
    }
    // ---- state gradient at the start of the sub-block --------------------------------------
    grad_step(R, dOt, Qt, aI, gI, I, w, g, tq, true);
    __syncthreads();   // staging and the tiny-gate list are complete

    // ---- exact gate gradients where the gate is too small for the cancelling form ----------
    //   dg_t[k] = (1/g_t) sum_d M[d] N[d],  M = S0[:,k] + sum_{i<t} Xt_i Kt_i[k],
    //                                       N = aI gI[k] R[:,k] + sum_{s>=t} dOt_s Qt_s[k]
    // (every term of N carries the factor g_t, so nothing cancels); d side with d and k exchanged.
    if (fix_n > 0) {
      const int n_fix = fix_n < kFixCap ? fix_n : kFixCap;
      if (fix_n > kFixCap && threadIdx.x == 0) atomicExch(rowflag + b, 1);   // let the scan kernels redo the row
      for (int e = w; e < n_fix; e += kThreads / 32) {
        const int code = fix_list[e];
        const bool dside = (code >> 16) != 0;
        const int t = (code >> 8) & 0xff, col = code & 0xff;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int o = lane + 32 * j;                 // index along the reduced axis
          const int d = dside ? col : o, kk = dside ? o : col;
          float M = S0[d * kLd + kk];
          for (int i = 0; i < t; ++i) M += Xt[(r0 + i) * kLd + d] * Kt[(r0 + i) * kLd + kk];
          float N = aIb[d] * gIb[kk] * Rm[d * kLd + kk];
          for (int s2 = t; s2 < kSub; ++s2) N += dOt[(r0 + s2) * kLd + d] * Qt[(r0 + s2) * kLd + kk];
          acc += M * N;
        }
        acc = warp_sum(acc);
        if (lane == 0) {
          const float *pre = dside ? Ap : Gp;
          const float cur = pre[(r0 + t) * kLd + col];
          const float prev = t > 0 ? pre[(r0 + t - 1) * kLd + col] : 1.f;
          T *tile = stg + (dside ? 4 : 2) * kSub * kStgLd;
          tile[t * kStgLd + col] = (T)(acc * prev / cur);
        }
      }
      __syncthreads();
    }

    // ---- coalesced write of the five 16 x 64 result tiles ----------------------------------
    {
      T *dst[5] = {dq, dk, dfk, dx, df};
#pragma unroll
      for (int it = 0; it < 5; ++it) {
        const int r = threadIdx.x >> 3, ch = threadIdx.x & 7;
        if (r0 + r < nvalid) {
          const uint4 val = *reinterpret_cast<const uint4 *>(stg + (it * kSub + r) * kStgLd + ch * 8);
          *reinterpret_cast<uint4 *>(dst[it] + base + (size_t)(r0 + r) * kDim + ch * 8) = val;
        }
      }
    }
    // the next iteration writes stg only after its own __syncthreads (after the state recompute)
  }
}

}  // namespace

size_t lfw_chunk_backward_scratch_bytes(int64_t B, int64_t T_) {
  const int64_t nc = ceil_div64(T_, kC);
  return align_up(bwd_scratch_floats(B, nc) * sizeof(float), 256);
}

template <typename T>
static int chunk_backward_typed(const void *go, const void *gs, const void *x, const void *f,
                                const void *q, const void *k, const void *fk, const void *state,
                                const void *ckpt, void *dx, void *df, void *dq, void *dk, void *dfk,
                                void *ds, int64_t B, int64_t T_, void *scratch, cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC);
  BwdScratch s = carve(scratch, B, nc);
  const size_t sm_local = (2 * kC * kLd + 2 * kNSub * kDim) * sizeof(float);
  const size_t sm_main = (6 * kC * kLd + 2 * kDim * kLd + 2 * kNSub * kSub * kLdP + 2 * kNSub * kDim +
                          4 * kDim + kDim + kFixCap) * sizeof(float) + 5 * kSub * kStgLd * sizeof(T);
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_chunk_bwd_main_kernel<T>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_main));
  if (umma_enabled()) {
    const int rc = lfw_chunk_local_umma(true, go, f, q, fk, s.G, s.Ac, s.Gc, s.flags, B, T_,
                                        std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
    if (rc != T2FW_OK) return rc;
  } else {
    lfw_chunk_bwd_local_kernel<T><<<(unsigned)(B * nc), kThreads, sm_local, st>>>(
        (const T *)go, (const T *)f, (const T *)q, (const T *)fk, s.G, s.Ac, s.Gc, s.flags, T_, nc);
    T2FW_CHECK_LAUNCH(1);
  }
  const int64_t n_carry = B * kDim * (kDim / 4);
  lfw_chunk_bwd_carry_kernel<T><<<(unsigned)ceil_div64(n_carry, 128), 128, 0, st>>>(
      (const T *)gs, s.G, s.Ac, s.Gc, s.flags, s.rowflag, (T *)ds, B, nc);
  T2FW_CHECK_LAUNCH(1);
  lfw_chunk_bwd_main_kernel<T><<<(unsigned)(B * nc), kThreads, sm_main, st>>>(
      (const T *)go, (const T *)x, (const T *)f, (const T *)q, (const T *)k, (const T *)fk,
      (const T *)state, (const T *)ckpt, s.G, (T *)dx, (T *)df, (T *)dq, (T *)dk, (T *)dfk,
      s.rowflag, T_, nc);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

int lfw_chunk_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                       const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
                       void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B, int64_t T_,
                       int dtype, void *scratch, cudaStream_t st, const int **rowflag_out) {
  const int64_t nc = ceil_div64(T_, kC);
  if (rowflag_out) *rowflag_out = carve(scratch, B, nc).rowflag;
  if (dtype == T2FW_F16)
    return chunk_backward_typed<__half>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds,
                                        B, T_, scratch, st);
  return chunk_backward_typed<__nv_bfloat16>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk,
                                             dfk, ds, B, T_, scratch, st);
}

}  // namespace t2fw
