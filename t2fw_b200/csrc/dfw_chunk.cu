// Delta rule in chunked form (D = M = 64, 16-bit storage): chunks of 64 steps, the contractions
// of a chunk on the tensor cores (mma.sync TF32, fp32 accumulation), the state carried in fp32.
//
// Replaces, for these shapes, the step-by-step scans of t2fw/csrc/dfw_kernel.cu:105-384.
//
// With K, Q [64 x M], V, dO [64 x D] the rows of one chunk, S0 the state before the chunk and
// L = strict_lower(K K^T):
//   delta rule per step:  d_t = v_t - S_{t-1} k_t,  S_t = S_{t-1} + d_t k_t^T,  o_t = S_{t-1} q_t
//   chunk form:           (I + L) Dl = V - K S0^T   =>  Dl = U - W S0^T,  W = (I+L)^-1 K,  U = (I+L)^-1 V
//                         O = Q S0^T + strict_lower(Q K^T) Dl ,   S_end = S0 + Dl^T K
// Backward (R = gradient of the state, walking the chunks in reverse; e_t = d_value_t = R_t k_t):
//                         (I + L^T) E = K R_end^T + strict_upper(K Q^T) dO
//                                   =>  E = Ub + Wb R_end^T,  Wb = (I+L^T)^-1 K,  Ub = (I+L^T)^-1 strict_upper(K Q^T) dO
//   d_value = E
//   d_query = dO S0 + strict_lower(dO Dl^T) K
//   d_key   = Dl R_end + strict_upper(Dl dO^T) Q - (strict_upper(X) + strict_lower(X^T)) K - E S0,   X = Dl E^T
//   R_start = R_end + dO^T Q - E^T K ,   S0 = S_end - Dl^T K   (the state is walked back from
//   final_state with the saved Dl, as the reference's backward does step by step)
//
// Kernels:
//   dfw_chunk_prep_kernel<T, kBwd>   (batch row, chunk): W, U (or Wb, Ub) by forward (backward)
//       substitution in fp32, one thread per column, no inverse is ever formed
//   dfw_chunk_fwd_kernel<T>          one CTA per batch row, sequential over chunks
//   dfw_chunk_bwd_seq_kernel<T>      one CTA per batch row, chunks in reverse: state walk-back, E, R
//   dfw_chunk_bwd_par_kernel<T>      (batch row, chunk): d_query and d_key from the stored S0, R_end, E
#include <type_traits>

#include "lfw_chunk.cuh"

namespace t2fw {

using namespace chunk;

namespace {

constexpr int kSeqThreads = 512;  // 16 warps: warp w owns rows 16*(w&3), columns 16*(w>>2) of a product
constexpr int kNT = 2;            // 8-column accumulator tiles per warp

// ---- prep: W, U (forward) or Wb, Ub (backward) --------------------------------------------------
// grid = B * nc, 128 threads (4 warps).  Output tiles are fp32 [64][64] row-major, rows beyond the
// end of the sequence are zero.  The Gram matrices K K^T and K Q^T come from the tensor cores and
// are exact up to fp32 summation order (16-bit inputs are exactly representable in TF32); the
// triangular solves run in fp32 on CUDA cores, one thread per right-hand-side column.
// warp w owns rows 16*w .. +15 of a 64 x 64 product
template <bool BT>
__device__ __forceinline__ void prep_gemm(float (&acc)[8][4], const float *tA, const float *tB, int m0, int g,
                                          int tq) {
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll 2
  for (int k0 = 0; k0 < kC; k0 += 8) {
    uint32_t a[4];
    lda(a, tA, kLd, m0, k0, g, tq);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      uint32_t bf[2];
      if (BT) ldb_t(bf, tB, kLd, k0, 8 * nt, g, tq); else ldb(bf, tB, kLd, k0, 8 * nt, g, tq);
      mma_tf32(acc[nt], a, bf);
    }
  }
}
// mode 0: store as is; 1: keep column > row, TF32-rounded (feeds an MMA)
template <int MODE>
__device__ __forceinline__ void prep_store(float *t, const float (&acc)[8][4], int m0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const int cc = 8 * nt + 2 * tq, r0 = m0 + g, r1 = m0 + g + 8;
    float v0 = acc[nt][0], v1 = acc[nt][1], v2 = acc[nt][2], v3 = acc[nt][3];
    if (MODE == 1) {
      v0 = (cc > r0) ? round_tf32(v0) : 0.f; v1 = (cc + 1 > r0) ? round_tf32(v1) : 0.f;
      v2 = (cc > r1) ? round_tf32(v2) : 0.f; v3 = (cc + 1 > r1) ? round_tf32(v3) : 0.f;
    }
    *reinterpret_cast<float2 *>(t + r0 * kLd + cc) = make_float2(v0, v1);
    *reinterpret_cast<float2 *>(t + r1 * kLd + cc) = make_float2(v2, v3);
  }
}

template <typename T, bool kBwd>
__global__ void __launch_bounds__(128)
dfw_chunk_prep_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v_or_go,
                      float *__restrict__ Wout, float *__restrict__ Uout, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Ks = sm, *Ls = Ks + kC * kLd, *Vs = Ls + kC * kLd, *Qs = Vs + kC * kLd;   // Qs: backward only
  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc, t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const size_t base = ((size_t)b * T_ + t0) * kDim;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;

  for (int idx = tid; idx < kC * (kDim / 2); idx += 128) {
    const int r = idx / (kDim / 2), c2 = (idx % (kDim / 2)) * 2;
    float2 kk = make_float2(0.f, 0.f), vv = kk, qq = kk;
    if (r < nvalid) {
      kk = Pair<T>::ld(k + base + (size_t)r * kDim + c2);
      vv = Pair<T>::ld(v_or_go + base + (size_t)r * kDim + c2);
      if (kBwd) qq = Pair<T>::ld(q + base + (size_t)r * kDim + c2);
    }
    *reinterpret_cast<float2 *>(Ks + r * kLd + c2) = kk;
    *reinterpret_cast<float2 *>(Vs + r * kLd + c2) = vv;
    if (kBwd) *reinterpret_cast<float2 *>(Qs + r * kLd + c2) = qq;
  }
  __syncthreads();

  float acc[8][4];
  // Ls[t][s] = k_t . k_s  (forward uses s < t, backward s > t)
  prep_gemm<true>(acc, Ks, Ks, 16 * w, g, tq);
  prep_store<0>(Ls, acc, 16 * w, g, tq);
  if (kBwd) {
    // right-hand side of the d side: rhs[t][d] = sum_{s>t} (k_t . q_s) dO[s][d]
    prep_gemm<true>(acc, Ks, Qs, 16 * w, g, tq);
    __syncthreads();                         // every warp has read Q
    prep_store<1>(Qs, acc, 16 * w, g, tq);   // strict upper part of K Q^T
    __syncthreads();
    prep_gemm<false>(acc, Qs, Vs, 16 * w, g, tq);
    __syncthreads();                         // every warp has read the scores
    prep_store<0>(Qs, acc, 16 * w, g, tq);   // rhs
  }
  __syncthreads();

  // substitution: thread = one column of [K | V] (forward) or [K | rhs] (backward)
  const int col = tid & 63;
  const bool second = tid >= 64;
  const float *rhs = second ? (kBwd ? Qs : Vs) : Ks;
  float x[kC];
  if (!kBwd) {
#pragma unroll
    for (int t = 0; t < kC; ++t) {
      float a0 = rhs[t * kLd + col], a1 = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < t; i4 += 4) {
        const float4 l4 = *reinterpret_cast<const float4 *>(Ls + t * kLd + i4);
        a0 = fmaf(-l4.x, x[i4], a0);
        if (i4 + 1 < t) a1 = fmaf(-l4.y, x[i4 + 1], a1);
        if (i4 + 2 < t) a0 = fmaf(-l4.z, x[i4 + 2], a0);
        if (i4 + 3 < t) a1 = fmaf(-l4.w, x[i4 + 3], a1);
      }
      x[t] = a0 + a1;
    }
  } else {
#pragma unroll
    for (int t = kC - 1; t >= 0; --t) {
      float a0 = rhs[t * kLd + col], a1 = 0.f;
#pragma unroll
      for (int s4 = ((t + 1) & ~3); s4 < kC; s4 += 4) {
        const float4 l4 = *reinterpret_cast<const float4 *>(Ls + t * kLd + s4);
        if (s4 > t) a0 = fmaf(-l4.x, x[s4], a0);
        if (s4 + 1 > t) a1 = fmaf(-l4.y, x[s4 + 1], a1);
        if (s4 + 2 > t) a0 = fmaf(-l4.z, x[s4 + 2], a0);
        if (s4 + 3 > t) a1 = fmaf(-l4.w, x[s4 + 3], a1);
      }
      x[t] = a0 + a1;
    }
  }
  float *dst = (second ? Uout : Wout) + (size_t)blockIdx.x * kC * kDim + col;
#pragma unroll
  for (int t = 0; t < kC; ++t) dst[t * kDim] = x[t];
}

// ---- helpers of the sequential kernels -------------------------------------------------------------
// acc[nt][.] (rows m0 + {g, g+8}, columns n0 + 8*nt + {2tq, 2tq+1}) += A * B over a contraction of 64.
//   AT: the tile holds A transposed (A[m][k] = tA[k][m]);  BT: the tile holds B as [n][k]
template <bool AT, bool BT>
__device__ __forceinline__ void gemm64(float (&acc)[kNT][4], const float *tA, const float *tB, int m0, int n0,
                                       int g, int tq) {
#pragma unroll 2
  for (int k0 = 0; k0 < kC; k0 += 8) {
    uint32_t a[4];
    if (AT) lda_t(a, tA, kLd, m0, k0, g, tq); else lda(a, tA, kLd, m0, k0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      uint32_t bf[2];
      if (BT) ldb_t(bf, tB, kLd, k0, n0 + 8 * nt, g, tq); else ldb(bf, tB, kLd, k0, n0 + 8 * nt, g, tq);
      mma_tf32(acc[nt], a, bf);
    }
  }
}
__device__ __forceinline__ void zero(float (&acc)[kNT][4]) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
}
// accumulator fragment -> fp32 tile (values rounded to TF32 so that the tile can feed an MMA)
__device__ __forceinline__ void store_acc(float *t, const float (&acc)[kNT][4], int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    *reinterpret_cast<float2 *>(t + (m0 + g) * kLd + cc) = make_float2(round_tf32(acc[nt][0]), round_tf32(acc[nt][1]));
    *reinterpret_cast<float2 *>(t + (m0 + g + 8) * kLd + cc) = make_float2(round_tf32(acc[nt][2]), round_tf32(acc[nt][3]));
  }
}
// Global loads are split in two, so that the loads of the next chunk are in flight while the
// current chunk is computed: piece `tid` of the 512 16-byte pieces of a 16-bit block ...
static_assert(kSeqThreads == 512, "one 16-byte piece of a 16-bit block per thread");
template <typename T>
__device__ __forceinline__ uint4 fetch16(const T *src, int nvalid, int tid) {
  const int r = tid >> 3, c8 = (tid & 7) * 8;
  return r < nvalid ? *reinterpret_cast<const uint4 *>(src + (size_t)r * kDim + c8) : make_uint4(0u, 0u, 0u, 0u);
}
template <typename T>
__device__ __forceinline__ void commit16(float *t, const uint4 &u, int tid) {
  const int r = tid >> 3, c8 = (tid & 7) * 8;
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  float vals[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 p = Pair<T>::ld(reinterpret_cast<const T *>(&w[j]));
    vals[2 * j] = round_tf32(p.x);
    vals[2 * j + 1] = round_tf32(p.y);
  }
  *reinterpret_cast<float4 *>(t + r * kLd + c8) = make_float4(vals[0], vals[1], vals[2], vals[3]);
  *reinterpret_cast<float4 *>(t + r * kLd + c8 + 4) = make_float4(vals[4], vals[5], vals[6], vals[7]);
}
// ... and pieces `tid`, `tid + 512` of the 1024 16-byte pieces of an fp32 block
__device__ __forceinline__ void fetch32(float4 (&r)[2], const float *src, int nrows, int tid) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int idx = tid + kSeqThreads * j, row = idx >> 4, c4 = (idx & 15) * 4;
    r[j] = row < nrows ? *reinterpret_cast<const float4 *>(src + (size_t)row * kDim + c4)
                       : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}
__device__ __forceinline__ void commit32(float *t, const float4 (&r)[2], int tid) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int idx = tid + kSeqThreads * j, row = idx >> 4, c4 = (idx & 15) * 4;
    *reinterpret_cast<float4 *>(t + row * kLd + c4) =
        make_float4(round_tf32(r[j].x), round_tf32(r[j].y), round_tf32(r[j].z), round_tf32(r[j].w));
  }
}
// this thread's accumulator-fragment positions of an fp32 [64][64] block
__device__ __forceinline__ void fetch_frag(float2 (&r)[kNT][2], const float *src, int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    r[nt][0] = *reinterpret_cast<const float2 *>(src + (size_t)(m0 + g) * kDim + cc);
    r[nt][1] = *reinterpret_cast<const float2 *>(src + (size_t)(m0 + g + 8) * kDim + cc);
  }
}

// ---- forward: one CTA per batch row, chunks in order ---------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kSeqThreads, 1)
dfw_chunk_fwd_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ state,
                     const float *__restrict__ W, const float *__restrict__ U, T *__restrict__ out,
                     T *__restrict__ final_state, float *__restrict__ delta, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Qs = sm, *Ks = Qs + kC * kLd, *Ws = Ks + kC * kLd, *Ds = Ws + kC * kLd, *Ss = Ds + kC * kLd,
        *As = Ss + kC * kLd;
  const int64_t b = blockIdx.x;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int m0 = 16 * (w & 3), n0 = 8 * kNT * (w >> 2);

  // the state: this warp's 16 x 32 tile in accumulator-fragment layout, fp32
  float S[kNT][4];
  {
    const T *sp = state + (size_t)b * kDim * kDim;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      const float2 lo = Pair<T>::ld(sp + (m0 + g) * kDim + cc), hi = Pair<T>::ld(sp + (m0 + g + 8) * kDim + cc);
      S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
    }
  }
  // global loads of a chunk, into registers: issued one chunk ahead
  uint4 rq, rk;
  float4 rw[2];
  float2 ru[kNT][2];
  auto fetch = [&](int64_t c) {
    const int64_t t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = ((size_t)b * nc + c) * kC * kDim;
    rq = fetch16<T>(q + base, nv, tid);
    rk = fetch16<T>(k + base, nv, tid);
    fetch32(rw, W + tile, kC, tid);
    fetch_frag(ru, U + tile, m0, n0, g, tq);
  };
  fetch(0);
  for (int64_t c = 0; c < nc; ++c) {
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim;
    commit16<T>(Qs, rq, tid);
    commit16<T>(Ks, rk, tid);
    commit32(Ws, rw, tid);
    float2 uf[kNT][2];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) { uf[nt][0] = ru[nt][0]; uf[nt][1] = ru[nt][1]; }
    store_acc(Ss, S, m0, n0, g, tq);
    __syncthreads();
    if (c + 1 < nc) fetch(c + 1);

    float acc[kNT][4], accO[kNT][4];
    // Dl = U - W S^T   (rows t, columns d)
    zero(acc);
    gemm64<false, true>(acc, Ws, Ss, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      const float2 u0 = uf[nt][0], u1 = uf[nt][1];
      acc[nt][0] = u0.x - acc[nt][0]; acc[nt][1] = u0.y - acc[nt][1];
      acc[nt][2] = u1.x - acc[nt][2]; acc[nt][3] = u1.y - acc[nt][3];
      if (m0 + g < nvalid)
        *reinterpret_cast<float2 *>(delta + base + (size_t)(m0 + g) * kDim + cc) = make_float2(acc[nt][0], acc[nt][1]);
      if (m0 + g + 8 < nvalid)
        *reinterpret_cast<float2 *>(delta + base + (size_t)(m0 + g + 8) * kDim + cc) = make_float2(acc[nt][2], acc[nt][3]);
    }
    // scores A = strict_lower(Q K^T)   (rows t, columns i)
    float sc[kNT][4];
    zero(sc);
    gemm64<false, true>(sc, Qs, Ks, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      sc[nt][0] = (cc < m0 + g) ? sc[nt][0] : 0.f;
      sc[nt][1] = (cc + 1 < m0 + g) ? sc[nt][1] : 0.f;
      sc[nt][2] = (cc < m0 + g + 8) ? sc[nt][2] : 0.f;
      sc[nt][3] = (cc + 1 < m0 + g + 8) ? sc[nt][3] : 0.f;
    }
    // O = Q S^T ...
    zero(accO);
    gemm64<false, true>(accO, Qs, Ss, m0, n0, g, tq);
    store_acc(Ds, acc, m0, n0, g, tq);
    store_acc(As, sc, m0, n0, g, tq);
    __syncthreads();
    // ... + A Dl
    gemm64<false, false>(accO, As, Ds, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      if (m0 + g < nvalid) Pair<T>::st(out + base + (size_t)(m0 + g) * kDim + cc, accO[nt][0], accO[nt][1]);
      if (m0 + g + 8 < nvalid) Pair<T>::st(out + base + (size_t)(m0 + g + 8) * kDim + cc, accO[nt][2], accO[nt][3]);
    }
    // S += Dl^T K   (rows d, columns m)
    gemm64<true, false>(S, Ds, Ks, m0, n0, g, tq);
    __syncthreads();               // tiles are rewritten by the next chunk
  }
  T *fp = final_state + (size_t)b * kDim * kDim;
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    Pair<T>::st(fp + (m0 + g) * kDim + cc, S[nt][0], S[nt][1]);
    Pair<T>::st(fp + (m0 + g + 8) * kDim + cc, S[nt][2], S[nt][3]);
  }
}

// this thread's accumulator-fragment positions -> fp32 [64][64] block in global memory
__device__ __forceinline__ void store_frag(float *dst, const float (&acc)[kNT][4], int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    *reinterpret_cast<float2 *>(dst + (size_t)(m0 + g) * kDim + cc) = make_float2(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<float2 *>(dst + (size_t)(m0 + g + 8) * kDim + cc) = make_float2(acc[nt][2], acc[nt][3]);
  }
}

// ---- backward, sequential part: one CTA per batch row, chunks in reverse ------------------------
// Only what depends on the chunk after it: the walked-back state S0, E = d_value and the state
// gradient R.  S0, R_end and E of every chunk go to scratch for the chunk-parallel kernel below.
template <typename T>
__global__ void __launch_bounds__(kSeqThreads, 1)
dfw_chunk_bwd_seq_kernel(const T *__restrict__ go, const T *__restrict__ gs, const T *__restrict__ q,
                         const T *__restrict__ k, const float *__restrict__ delta,
                         const T *__restrict__ final_state, const float *__restrict__ Wb,
                         const float *__restrict__ Ub, float *__restrict__ Sc, float *__restrict__ Rc,
                         float *__restrict__ Ec, T *__restrict__ dv, T *__restrict__ ds, int64_t T_,
                         int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Qs = sm, *Ks = Qs + kC * kLd, *Gs = Ks + kC * kLd, *Ds = Gs + kC * kLd, *Ws = Ds + kC * kLd,
        *Es = Ws + kC * kLd, *Rs = Es + kC * kLd;
  const int64_t b = blockIdx.x;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int m0 = 16 * (w & 3), n0 = 8 * kNT * (w >> 2);

  float R[kNT][4], S[kNT][4];     // state gradient and state (walked back), fp32 fragments
  {
    const T *rp = gs + (size_t)b * kDim * kDim, *sp = final_state + (size_t)b * kDim * kDim;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      float2 lo = Pair<T>::ld(rp + (m0 + g) * kDim + cc), hi = Pair<T>::ld(rp + (m0 + g + 8) * kDim + cc);
      R[nt][0] = lo.x; R[nt][1] = lo.y; R[nt][2] = hi.x; R[nt][3] = hi.y;
      lo = Pair<T>::ld(sp + (m0 + g) * kDim + cc); hi = Pair<T>::ld(sp + (m0 + g + 8) * kDim + cc);
      S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
    }
  }
  // global loads of a chunk, into registers: issued one chunk ahead
  uint4 rq, rk, rg;
  float4 rd[2], rw[2];
  float2 ru[kNT][2];
  auto fetch = [&](int64_t c) {
    const int64_t t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = ((size_t)b * nc + c) * kC * kDim;
    rq = fetch16<T>(q + base, nv, tid);
    rk = fetch16<T>(k + base, nv, tid);
    rg = fetch16<T>(go + base, nv, tid);
    fetch32(rd, delta + base, nv, tid);
    fetch32(rw, Wb + tile, kC, tid);
    fetch_frag(ru, Ub + tile, m0, n0, g, tq);
  };
  fetch(nc - 1);
  for (int64_t c = nc - 1; c >= 0; --c) {
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = ((size_t)b * nc + c) * kC * kDim;
    commit16<T>(Qs, rq, tid);
    commit16<T>(Ks, rk, tid);
    commit16<T>(Gs, rg, tid);
    commit32(Ds, rd, tid);
    commit32(Ws, rw, tid);
    float2 uf[kNT][2];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) { uf[nt][0] = ru[nt][0]; uf[nt][1] = ru[nt][1]; }
    store_acc(Rs, R, m0, n0, g, tq);
    store_frag(Rc + tile, R, m0, n0, g, tq);
    __syncthreads();
    if (c > 0) fetch(c - 1);

    float acc[kNT][4];
    // S0 = S_end - Dl^T K
    zero(acc);
    gemm64<true, false>(acc, Ds, Ks, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[nt][e] -= acc[nt][e];
    store_frag(Sc + tile, S, m0, n0, g, tq);
    // E = Ub + Wb R_end^T = d_value
    zero(acc);
    gemm64<false, true>(acc, Ws, Rs, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      const float2 u0 = uf[nt][0], u1 = uf[nt][1];
      acc[nt][0] += u0.x; acc[nt][1] += u0.y; acc[nt][2] += u1.x; acc[nt][3] += u1.y;
      if (m0 + g < nvalid) Pair<T>::st(dv + base + (size_t)(m0 + g) * kDim + cc, acc[nt][0], acc[nt][1]);
      if (m0 + g + 8 < nvalid) Pair<T>::st(dv + base + (size_t)(m0 + g + 8) * kDim + cc, acc[nt][2], acc[nt][3]);
    }
    store_acc(Es, acc, m0, n0, g, tq);
    store_frag(Ec + tile, acc, m0, n0, g, tq);
    __syncthreads();               // E tile complete
    // R_start = R_end + dO^T Q - E^T K
    gemm64<true, false>(R, Gs, Qs, m0, n0, g, tq);
    zero(acc);
    gemm64<true, false>(acc, Es, Ks, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) R[nt][e] -= acc[nt][e];
    __syncthreads();               // tiles are rewritten by the next chunk
  }
  T *dp = ds + (size_t)b * kDim * kDim;
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    Pair<T>::st(dp + (m0 + g) * kDim + cc, R[nt][0], R[nt][1]);
    Pair<T>::st(dp + (m0 + g + 8) * kDim + cc, R[nt][2], R[nt][3]);
  }
}

// ---- backward, chunk-parallel part: d_query and d_key of one (batch row, chunk) ------------------
template <typename T>
__global__ void __launch_bounds__(kSeqThreads, 1)
dfw_chunk_bwd_par_kernel(const T *__restrict__ go, const T *__restrict__ q, const T *__restrict__ k,
                         const float *__restrict__ delta, const float *__restrict__ Sc,
                         const float *__restrict__ Rc, const float *__restrict__ Ec, T *__restrict__ dq,
                         T *__restrict__ dk, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Qs = sm, *Ks = Qs + kC * kLd, *Gs = Ks + kC * kLd, *Ds = Gs + kC * kLd, *Es = Ds + kC * kLd,
        *Rs = Es + kC * kLd, *Ss = Rs + kC * kLd, *X1s = Ss + kC * kLd, *X2s = X1s + kC * kLd;
  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc, t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const size_t base = ((size_t)b * T_ + t0) * kDim, tile = (size_t)blockIdx.x * kC * kDim;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int m0 = 16 * (w & 3), n0 = 8 * kNT * (w >> 2);
  {
    const uint4 rq = fetch16<T>(q + base, nvalid, tid), rk = fetch16<T>(k + base, nvalid, tid),
                rg = fetch16<T>(go + base, nvalid, tid);
    float4 rd[2], re[2], rs[2], rr[2];
    fetch32(rd, delta + base, nvalid, tid);
    fetch32(re, Ec + tile, kC, tid);
    fetch32(rs, Sc + tile, kC, tid);
    fetch32(rr, Rc + tile, kC, tid);
    commit16<T>(Qs, rq, tid);
    commit16<T>(Ks, rk, tid);
    commit16<T>(Gs, rg, tid);
    commit32(Ds, rd, tid);
    commit32(Es, re, tid);
    commit32(Ss, rs, tid);
    commit32(Rs, rr, tid);
  }
  __syncthreads();
  float acc[kNT][4], acc2[kNT][4];
  // X1 = strict_lower(dO Dl^T)
  zero(acc);
  gemm64<false, true>(acc, Gs, Ds, m0, n0, g, tq);
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    acc[nt][0] = (cc < m0 + g) ? acc[nt][0] : 0.f;
    acc[nt][1] = (cc + 1 < m0 + g) ? acc[nt][1] : 0.f;
    acc[nt][2] = (cc < m0 + g + 8) ? acc[nt][2] : 0.f;
    acc[nt][3] = (cc + 1 < m0 + g + 8) ? acc[nt][3] : 0.f;
  }
  store_acc(X1s, acc, m0, n0, g, tq);
  // X2 = strict_upper(Dl E^T)
  zero(acc);
  gemm64<false, true>(acc, Ds, Es, m0, n0, g, tq);
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    acc[nt][0] = (cc > m0 + g) ? acc[nt][0] : 0.f;
    acc[nt][1] = (cc + 1 > m0 + g) ? acc[nt][1] : 0.f;
    acc[nt][2] = (cc > m0 + g + 8) ? acc[nt][2] : 0.f;
    acc[nt][3] = (cc + 1 > m0 + g + 8) ? acc[nt][3] : 0.f;
  }
  store_acc(X2s, acc, m0, n0, g, tq);
  // d_query = dO S0 + X1 K ;  d_key = Dl R_end + X1^T Q - (X2 + X2^T) K - E S0
  zero(acc);
  gemm64<false, false>(acc, Gs, Ss, m0, n0, g, tq);
  zero(acc2);
  gemm64<false, false>(acc2, Es, Ss, m0, n0, g, tq);
  float acck[kNT][4];
  zero(acck);
  gemm64<false, false>(acck, Ds, Rs, m0, n0, g, tq);
  __syncthreads();                 // X1, X2 tiles complete
  gemm64<false, false>(acc, X1s, Ks, m0, n0, g, tq);
  gemm64<true, false>(acck, X1s, Qs, m0, n0, g, tq);
  gemm64<false, false>(acc2, X2s, Ks, m0, n0, g, tq);
  gemm64<true, false>(acc2, X2s, Ks, m0, n0, g, tq);
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    if (m0 + g < nvalid) {
      Pair<T>::st(dq + base + (size_t)(m0 + g) * kDim + cc, acc[nt][0], acc[nt][1]);
      Pair<T>::st(dk + base + (size_t)(m0 + g) * kDim + cc, acck[nt][0] - acc2[nt][0], acck[nt][1] - acc2[nt][1]);
    }
    if (m0 + g + 8 < nvalid) {
      Pair<T>::st(dq + base + (size_t)(m0 + g + 8) * kDim + cc, acc[nt][2], acc[nt][3]);
      Pair<T>::st(dk + base + (size_t)(m0 + g + 8) * kDim + cc, acck[nt][2] - acc2[nt][2], acck[nt][3] - acc2[nt][3]);
    }
  }
}

constexpr size_t kTileBytes = (size_t)kC * kLd * sizeof(float);
constexpr size_t kPrepTile = kTileBytes;

inline size_t wu_floats(int64_t B, int64_t nc) { return (size_t)B * nc * kC * kDim; }

}  // namespace

bool dfw_chunk_supported(int64_t D, int64_t M, int dtype) {
  return D == kDim && M == kDim && (dtype == T2FW_F16 || dtype == T2FW_BF16);
}

// fp32 [B][n_chunks][64][64] arrays: W and U (forward); Wb, Ub and the per-chunk S0, R_end, E (backward)
size_t dfw_chunk_scratch_bytes(int64_t B, int64_t T_, bool backward) {
  return align_up((backward ? 5 : 2) * wu_floats(B, ceil_div64(T_, kC)) * sizeof(float), 256);
}

template <typename T>
static int dfw_chunk_forward_typed(const void *q, const void *k, const void *v, const void *state, void *out,
                                   void *final_state, void *delta, int64_t B, int64_t T_, void *scratch,
                                   cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC);
  float *W = static_cast<float *>(scratch), *U = W + wu_floats(B, nc);
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_prep_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(3 * kPrepTile)));
  dfw_chunk_prep_kernel<T, false><<<(unsigned)(B * nc), 128, 3 * kPrepTile, st>>>(
      (const T *)q, (const T *)k, (const T *)v, W, U, T_, nc);
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(6 * kTileBytes)));
  dfw_chunk_fwd_kernel<T><<<(unsigned)B, kSeqThreads, 6 * kTileBytes, st>>>(
      (const T *)q, (const T *)k, (const T *)state, W, U, (T *)out, (T *)final_state, (float *)delta, T_, nc);
  T2FW_CHECK_LAUNCH(2);
  return T2FW_OK;
}

int dfw_chunk_forward(const void *q, const void *k, const void *v, const void *state, void *out,
                      void *final_state, void *delta, int64_t B, int64_t T_, int dtype, void *scratch,
                      cudaStream_t st) {
  if (dtype == T2FW_F16)
    return dfw_chunk_forward_typed<__half>(q, k, v, state, out, final_state, delta, B, T_, scratch, st);
  return dfw_chunk_forward_typed<__nv_bfloat16>(q, k, v, state, out, final_state, delta, B, T_, scratch, st);
}

template <typename T>
static int dfw_chunk_backward_typed(const void *go, const void *gs, const void *q, const void *k,
                                    const void *delta, const void *final_state, void *dq, void *dk, void *dv,
                                    void *ds, int64_t B, int64_t T_, void *scratch, cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC);
  float *Wb = static_cast<float *>(scratch), *Ub = Wb + wu_floats(B, nc);
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_prep_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(4 * kPrepTile)));
  dfw_chunk_prep_kernel<T, true><<<(unsigned)(B * nc), 128, 4 * kPrepTile, st>>>(
      (const T *)q, (const T *)k, (const T *)go, Wb, Ub, T_, nc);
  float *Sc = Ub + wu_floats(B, nc), *Rc = Sc + wu_floats(B, nc), *Ec = Rc + wu_floats(B, nc);
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_bwd_seq_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(7 * kTileBytes)));
  dfw_chunk_bwd_seq_kernel<T><<<(unsigned)B, kSeqThreads, 7 * kTileBytes, st>>>(
      (const T *)go, (const T *)gs, (const T *)q, (const T *)k, (const float *)delta, (const T *)final_state, Wb,
      Ub, Sc, Rc, Ec, (T *)dv, (T *)ds, T_, nc);
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_bwd_par_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(9 * kTileBytes)));
  dfw_chunk_bwd_par_kernel<T><<<(unsigned)(B * nc), kSeqThreads, 9 * kTileBytes, st>>>(
      (const T *)go, (const T *)q, (const T *)k, (const float *)delta, Sc, Rc, Ec, (T *)dq, (T *)dk, T_, nc);
  T2FW_CHECK_LAUNCH(3);
  return T2FW_OK;
}

int dfw_chunk_backward(const void *go, const void *gs, const void *q, const void *k, const void *delta,
                       const void *final_state, void *dq, void *dk, void *dv, void *ds, int64_t B, int64_t T_,
                       int dtype, void *scratch, cudaStream_t st) {
  if (dtype == T2FW_F16)
    return dfw_chunk_backward_typed<__half>(go, gs, q, k, delta, final_state, dq, dk, dv, ds, B, T_, scratch, st);
  return dfw_chunk_backward_typed<__nv_bfloat16>(go, gs, q, k, delta, final_state, dq, dk, dv, ds, B, T_, scratch,
                                                 st);
}

}  // namespace t2fw
