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
// The last three have tcgen05 versions in dfw_chunk_umma.cu, which the launchers below prefer; the
// versions here run when a pointer is not 16-byte aligned or T2FW_DISABLE_DFW_UMMA=1 is set.
#include <cstdlib>
#include <type_traits>

#include "lfw_chunk.cuh"

namespace t2fw {

using namespace chunk;

namespace {

constexpr int kSeqThreads = 512;  // 16 warps: warp w owns rows 16*(w&3), columns 16*(w>>2) of a product
constexpr int kNT = 2;            // 8-column accumulator tiles per warp
// U and Ub tiles (the right-hand sides after substitution) are stored with rows of kLdU = 68 floats:
// a tile then lands in shared memory by one bulk copy with its rows 17 x 16 bytes apart, which
// lets threads that own consecutive rows read 16-byte pieces without bank conflicts
constexpr int kLdU = kDim + 4;

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

  // 512 16-byte pieces per [64][64] block, 4 per thread and tensor; all loads are issued before
  // the first conversion so that their latencies overlap
  {
    uint4 rk[4], rv[4], rq[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = tid + 128 * j, r = idx >> 3, c8 = (idx & 7) * 8;
      const bool in = r < nvalid;
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      rk[j] = in ? *reinterpret_cast<const uint4 *>(k + base + (size_t)r * kDim + c8) : z;
      rv[j] = in ? *reinterpret_cast<const uint4 *>(v_or_go + base + (size_t)r * kDim + c8) : z;
      if (kBwd) rq[j] = in ? *reinterpret_cast<const uint4 *>(q + base + (size_t)r * kDim + c8) : z;
    }
    auto put = [&](float *t, const uint4 &u, int idx) {
      const int r = idx >> 3, c8 = (idx & 7) * 8;
      const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
      float vals[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 p2 = Pair<T>::ld(reinterpret_cast<const T *>(&w4[e]));
        vals[2 * e] = p2.x;
        vals[2 * e + 1] = p2.y;
      }
      *reinterpret_cast<float4 *>(t + r * kLd + c8) = make_float4(vals[0], vals[1], vals[2], vals[3]);
      *reinterpret_cast<float4 *>(t + r * kLd + c8 + 4) = make_float4(vals[4], vals[5], vals[6], vals[7]);
    };
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      put(Ks, rk[j], tid + 128 * j);
      put(Vs, rv[j], tid + 128 * j);
      if (kBwd) put(Qs, rq[j], tid + 128 * j);
    }
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
  // the second tile has its rows padded to kLdU floats (see kLdU)
  const int ld = second ? kLdU : kDim;
  float *dst = (second ? Uout : Wout) + (size_t)blockIdx.x * kC * ld + col;
#pragma unroll
  for (int t = 0; t < kC; ++t) dst[t * ld] = x[t];
}

// ---- helpers of the chunk kernels ----------------------------------------------------------------
// Every product has the form D[m][n] = sum_k A[m][k] B[n][k] with both tiles stored [row][k];
// operands that arise the other way round are stored transposed at the moment they are written.
// Within 16 values of k, thread tq of a fragment group uses the physical columns 4tq .. 4tq+3 for
// the logical k indices (tq, tq+4) of two consecutive MMAs - the sum over k does not depend on
// the order as long as A and B agree - so every fragment is one 16-byte load.
constexpr int kLdV = 80;   // row stride in floats: the 16-byte loads of a quarter warp hit 32 distinct banks

__device__ __forceinline__ void gemm64(float (&acc)[kNT][4], const float *tA, const float *tB, int m0, int n0,
                                       int g, int tq) {
#pragma unroll
  for (int k0 = 0; k0 < kC; k0 += 16) {
    const float4 lo = *reinterpret_cast<const float4 *>(tA + (m0 + g) * kLdV + k0 + 4 * tq);
    const float4 hi = *reinterpret_cast<const float4 *>(tA + (m0 + g + 8) * kLdV + k0 + 4 * tq);
    const uint32_t a1[4] = {__float_as_uint(lo.x), __float_as_uint(hi.x), __float_as_uint(lo.y), __float_as_uint(hi.y)};
    const uint32_t a2[4] = {__float_as_uint(lo.z), __float_as_uint(hi.z), __float_as_uint(lo.w), __float_as_uint(hi.w)};
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const float4 bv = *reinterpret_cast<const float4 *>(tB + (n0 + 8 * nt + g) * kLdV + k0 + 4 * tq);
      const uint32_t b1[2] = {__float_as_uint(bv.x), __float_as_uint(bv.y)};
      const uint32_t b2[2] = {__float_as_uint(bv.z), __float_as_uint(bv.w)};
      mma_tf32(acc[nt], a1, b1);
      mma_tf32(acc[nt], a2, b2);
    }
  }
}
__device__ __forceinline__ void zero(float (&acc)[kNT][4]) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
}
// keep the strictly lower (LOWER) or strictly upper part of this warp's accumulator tile
template <bool LOWER>
__device__ __forceinline__ void mask_tri(float (&acc)[kNT][4], int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq, r0 = m0 + g, r1 = m0 + g + 8;
    acc[nt][0] = (LOWER ? cc < r0 : cc > r0) ? acc[nt][0] : 0.f;
    acc[nt][1] = (LOWER ? cc + 1 < r0 : cc + 1 > r0) ? acc[nt][1] : 0.f;
    acc[nt][2] = (LOWER ? cc < r1 : cc > r1) ? acc[nt][2] : 0.f;
    acc[nt][3] = (LOWER ? cc + 1 < r1 : cc + 1 > r1) ? acc[nt][3] : 0.f;
  }
}
// accumulator fragment -> TF32 tile, as is ([m][n]) or transposed ([n][m])
__device__ __forceinline__ void store_acc(float *t, const float (&acc)[kNT][4], int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    *reinterpret_cast<float2 *>(t + (m0 + g) * kLdV + cc) = make_float2(round_tf32(acc[nt][0]), round_tf32(acc[nt][1]));
    *reinterpret_cast<float2 *>(t + (m0 + g + 8) * kLdV + cc) = make_float2(round_tf32(acc[nt][2]), round_tf32(acc[nt][3]));
  }
}
__device__ __forceinline__ void store_acc_t(float *t, const float (&acc)[kNT][4], int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    t[cc * kLdV + m0 + g] = round_tf32(acc[nt][0]);
    t[(cc + 1) * kLdV + m0 + g] = round_tf32(acc[nt][1]);
    t[cc * kLdV + m0 + g + 8] = round_tf32(acc[nt][2]);
    t[(cc + 1) * kLdV + m0 + g + 8] = round_tf32(acc[nt][3]);
  }
}
// accumulator fragment <-> fp32 [64][64] block in global memory, as is or transposed
__device__ __forceinline__ void store_frag(float *dst, const float (&acc)[kNT][4], int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    *reinterpret_cast<float2 *>(dst + (size_t)(m0 + g) * kDim + cc) = make_float2(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<float2 *>(dst + (size_t)(m0 + g + 8) * kDim + cc) = make_float2(acc[nt][2], acc[nt][3]);
  }
}
__device__ __forceinline__ void store_frag_t(float *dst, const float (&acc)[kNT][4], int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    dst[(size_t)cc * kDim + m0 + g] = acc[nt][0];
    dst[(size_t)(cc + 1) * kDim + m0 + g] = acc[nt][1];
    dst[(size_t)cc * kDim + m0 + g + 8] = acc[nt][2];
    dst[(size_t)(cc + 1) * kDim + m0 + g + 8] = acc[nt][3];
  }
}
// accumulator-fragment-shaped read of a U / Ub tile (rows padded to kLdU floats)
__device__ __forceinline__ void fetch_frag(float2 (&r)[kNT][2], const float *src, int m0, int n0, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    const int cc = n0 + 8 * nt + 2 * tq;
    r[nt][0] = *reinterpret_cast<const float2 *>(src + (size_t)(m0 + g) * kLdU + cc);
    r[nt][1] = *reinterpret_cast<const float2 *>(src + (size_t)(m0 + g + 8) * kLdU + cc);
  }
}

// Global loads are split in two (fetch into registers, commit to a shared-memory tile) so that the
// loads of the next chunk are in flight while the current chunk is computed.  A [64][64] block
// is 512 (16-bit) or 1024 (fp32) 16-byte pieces.  Piece mapping ROWS: consecutive threads take
// consecutive pieces of a row (coalesced; for tiles kept as they are).  Piece mapping COLS:
// consecutive threads take the same piece of consecutive rows, which makes the transposed
// shared-memory stores conflict-free (for tiles kept transposed).
static_assert(kSeqThreads == 512, "one 16-byte piece of a 16-bit block per thread");
template <typename T, bool COLS>
__device__ __forceinline__ uint4 fetch16(const T *src, int nvalid, int tid) {
  const int r = COLS ? (tid & 63) : (tid >> 3), c8 = (COLS ? (tid >> 6) : (tid & 7)) * 8;
  return r < nvalid ? *reinterpret_cast<const uint4 *>(src + (size_t)r * kDim + c8) : make_uint4(0u, 0u, 0u, 0u);
}
template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &u, float (&vals)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 p = Pair<T>::ld(reinterpret_cast<const T *>(&w[j]));
    vals[2 * j] = round_tf32(p.x);
    vals[2 * j + 1] = round_tf32(p.y);
  }
}
// commit as is ([row][col]); works with either piece mapping
template <typename T, bool COLS>
__device__ __forceinline__ void commit16(float *t, const uint4 &u, int tid) {
  const int r = COLS ? (tid & 63) : (tid >> 3), c8 = (COLS ? (tid >> 6) : (tid & 7)) * 8;
  float vals[8];
  unpack8<T>(u, vals);
  *reinterpret_cast<float4 *>(t + r * kLdV + c8) = make_float4(vals[0], vals[1], vals[2], vals[3]);
  *reinterpret_cast<float4 *>(t + r * kLdV + c8 + 4) = make_float4(vals[4], vals[5], vals[6], vals[7]);
}
// commit transposed ([col][row]); piece mapping COLS
template <typename T>
__device__ __forceinline__ void commit16_t(float *t, const uint4 &u, int tid) {
  const int r = tid & 63, c8 = (tid >> 6) * 8;
  float vals[8];
  unpack8<T>(u, vals);
#pragma unroll
  for (int j = 0; j < 8; ++j) t[(c8 + j) * kLdV + r] = vals[j];
}
template <bool COLS>
__device__ __forceinline__ void fetch32(float4 (&r)[2], const float *src, int nrows, int tid) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int idx = tid + kSeqThreads * j;
    const int row = COLS ? (idx & 63) : (idx >> 4), c4 = (COLS ? (idx >> 6) : (idx & 15)) * 4;
    r[j] = row < nrows ? *reinterpret_cast<const float4 *>(src + (size_t)row * kDim + c4)
                       : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}
__device__ __forceinline__ void commit32(float *t, const float4 (&r)[2], int tid) {    // mapping ROWS, as is
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int idx = tid + kSeqThreads * j, row = idx >> 4, c4 = (idx & 15) * 4;
    *reinterpret_cast<float4 *>(t + row * kLdV + c4) =
        make_float4(round_tf32(r[j].x), round_tf32(r[j].y), round_tf32(r[j].z), round_tf32(r[j].w));
  }
}
__device__ __forceinline__ void commit32_t(float *t, const float4 (&r)[2], int tid) {  // mapping COLS, transposed
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int idx = tid + kSeqThreads * j, row = idx & 63, c4 = (idx >> 6) * 4;
    t[c4 * kLdV + row] = round_tf32(r[j].x);
    t[(c4 + 1) * kLdV + row] = round_tf32(r[j].y);
    t[(c4 + 2) * kLdV + row] = round_tf32(r[j].z);
    t[(c4 + 3) * kLdV + row] = round_tf32(r[j].w);
  }
}

// ---- forward: one CTA per batch row, chunks in order ---------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kSeqThreads, 1)
dfw_chunk_fwd_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ state,
                     const float *__restrict__ W, const float *__restrict__ U, T *__restrict__ out,
                     T *__restrict__ final_state, float *__restrict__ delta, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  constexpr int kTileF = kC * kLdV;
  // Q [t][m], K [t][m], K^T [m][t], W [t][m], S [d][m], A = strict_lower(Q K^T) [t][i], Dl^T [d][t]
  float *Qs = sm, *Ks = Qs + kTileF, *KsT = Ks + kTileF, *Ws = KsT + kTileF, *Ss = Ws + kTileF,
        *As = Ss + kTileF, *DsT = As + kTileF;
  const int64_t b = blockIdx.x;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int m0 = 16 * (w & 3), n0 = 8 * kNT * (w >> 2);

  // the state: this warp's 16 x 16 tile in accumulator-fragment layout, fp32
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
    rq = fetch16<T, false>(q + base, nv, tid);
    rk = fetch16<T, true>(k + base, nv, tid);
    fetch32<false>(rw, W + tile, kC, tid);
    fetch_frag(ru, U + ((size_t)b * nc + c) * kC * kLdU, m0, n0, g, tq);
  };
  fetch(0);
  for (int64_t c = 0; c < nc; ++c) {
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim;
    commit16<T, false>(Qs, rq, tid);
    commit16<T, true>(Ks, rk, tid);
    commit16_t<T>(KsT, rk, tid);
    commit32(Ws, rw, tid);
    float2 uf[kNT][2];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) { uf[nt][0] = ru[nt][0]; uf[nt][1] = ru[nt][1]; }
    store_acc(Ss, S, m0, n0, g, tq);
    __syncthreads();
    if (c + 1 < nc) fetch(c + 1);

    float acc[kNT][4], accO[kNT][4], sc[kNT][4];
    // Dl = U - W S^T   (rows t, columns d)
    zero(acc);
    gemm64(acc, Ws, Ss, m0, n0, g, tq);
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
    store_acc_t(DsT, acc, m0, n0, g, tq);
    // scores A = strict_lower(Q K^T)   (rows t, columns i)
    zero(sc);
    gemm64(sc, Qs, Ks, m0, n0, g, tq);
    mask_tri<true>(sc, m0, n0, g, tq);
    store_acc(As, sc, m0, n0, g, tq);
    // O = Q S^T ...
    zero(accO);
    gemm64(accO, Qs, Ss, m0, n0, g, tq);
    __syncthreads();
    // ... + A Dl
    gemm64(accO, As, DsT, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      if (m0 + g < nvalid) Pair<T>::st(out + base + (size_t)(m0 + g) * kDim + cc, accO[nt][0], accO[nt][1]);
      if (m0 + g + 8 < nvalid) Pair<T>::st(out + base + (size_t)(m0 + g + 8) * kDim + cc, accO[nt][2], accO[nt][3]);
    }
    // S += Dl^T K   (rows d, columns m)
    gemm64(S, DsT, KsT, m0, n0, g, tq);
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

// ---- backward, sequential part: one CTA per batch row, chunks in reverse ------------------------
// Only what depends on the chunk after it: the walked-back state S0, E = d_value and the state
// gradient R.  S0^T, R_end^T and E of every chunk go to scratch for the chunk-parallel kernel below.
template <typename T>
__global__ void __launch_bounds__(kSeqThreads, 1)
dfw_chunk_bwd_seq_kernel(const T *__restrict__ go, const T *__restrict__ gs, const T *__restrict__ q,
                         const T *__restrict__ k, const float *__restrict__ delta,
                         const T *__restrict__ final_state, const float *__restrict__ Wb,
                         const float *__restrict__ Ub, float *__restrict__ ScT, float *__restrict__ RcT,
                         float *__restrict__ Ec, T *__restrict__ dv, T *__restrict__ ds, int64_t T_,
                         int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  constexpr int kTileF = kC * kLdV;
  // K^T [m][t], Q^T [m][t], dO^T [d][t], Dl^T [d][t], Wb [t][m], E^T [d][t], R [d][m]
  float *KsT = sm, *QsT = KsT + kTileF, *GsT = QsT + kTileF, *DsT = GsT + kTileF, *Ws = DsT + kTileF,
        *EsT = Ws + kTileF, *Rs = EsT + kTileF;
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
  uint4 rq, rk, rg;
  float4 rd[2], rw[2];
  float2 ru[kNT][2];
  auto fetch = [&](int64_t c) {
    const int64_t t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = ((size_t)b * nc + c) * kC * kDim;
    rq = fetch16<T, true>(q + base, nv, tid);
    rk = fetch16<T, true>(k + base, nv, tid);
    rg = fetch16<T, true>(go + base, nv, tid);
    fetch32<true>(rd, delta + base, nv, tid);
    fetch32<false>(rw, Wb + tile, kC, tid);
    fetch_frag(ru, Ub + ((size_t)b * nc + c) * kC * kLdU, m0, n0, g, tq);
  };
  fetch(nc - 1);
  for (int64_t c = nc - 1; c >= 0; --c) {
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = ((size_t)b * nc + c) * kC * kDim;
    commit16_t<T>(QsT, rq, tid);
    commit16_t<T>(KsT, rk, tid);
    commit16_t<T>(GsT, rg, tid);
    commit32_t(DsT, rd, tid);
    commit32(Ws, rw, tid);
    float2 uf[kNT][2];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) { uf[nt][0] = ru[nt][0]; uf[nt][1] = ru[nt][1]; }
    store_acc(Rs, R, m0, n0, g, tq);
    store_frag_t(RcT + tile, R, m0, n0, g, tq);
    __syncthreads();
    if (c > 0) fetch(c - 1);

    float acc[kNT][4];
    // S0 = S_end - Dl^T K
    zero(acc);
    gemm64(acc, DsT, KsT, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[nt][e] -= acc[nt][e];
    store_frag_t(ScT + tile, S, m0, n0, g, tq);
    // E = Ub + Wb R_end^T = d_value
    zero(acc);
    gemm64(acc, Ws, Rs, m0, n0, g, tq);
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      const int cc = n0 + 8 * nt + 2 * tq;
      const float2 u0 = uf[nt][0], u1 = uf[nt][1];
      acc[nt][0] += u0.x; acc[nt][1] += u0.y; acc[nt][2] += u1.x; acc[nt][3] += u1.y;
      if (m0 + g < nvalid) Pair<T>::st(dv + base + (size_t)(m0 + g) * kDim + cc, acc[nt][0], acc[nt][1]);
      if (m0 + g + 8 < nvalid) Pair<T>::st(dv + base + (size_t)(m0 + g + 8) * kDim + cc, acc[nt][2], acc[nt][3]);
    }
    store_acc_t(EsT, acc, m0, n0, g, tq);
    store_frag(Ec + tile, acc, m0, n0, g, tq);
    __syncthreads();               // E^T tile complete
    // R_start = R_end + dO^T Q - E^T K
    gemm64(R, GsT, QsT, m0, n0, g, tq);
    zero(acc);
    gemm64(acc, EsT, KsT, m0, n0, g, tq);
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
                         const float *__restrict__ delta, const float *__restrict__ ScT,
                         const float *__restrict__ RcT, const float *__restrict__ Ec, T *__restrict__ dq,
                         T *__restrict__ dk, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  constexpr int kTileF = kC * kLdV;
  // dO [t][d], Dl [t][d], E [t][d], S0^T [m][d], R_end^T [m][d], K^T [m][t], Q^T [m][t],
  // X1 = strict_lower(dO Dl^T) [t][i] and its transpose, Y = strict_upper(X2) + its mirror image, X2 = Dl E^T
  float *Gs = sm, *Ds = Gs + kTileF, *Es = Ds + kTileF, *SsT = Es + kTileF, *RsT = SsT + kTileF,
        *KsT = RsT + kTileF, *QsT = KsT + kTileF, *X1s = QsT + kTileF, *X1sT = X1s + kTileF, *Ys = X1sT + kTileF;
  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc, t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const size_t base = ((size_t)b * T_ + t0) * kDim, tile = (size_t)blockIdx.x * kC * kDim;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int m0 = 16 * (w & 3), n0 = 8 * kNT * (w >> 2);
  {
    const uint4 rq = fetch16<T, true>(q + base, nvalid, tid), rk = fetch16<T, true>(k + base, nvalid, tid),
                rg = fetch16<T, false>(go + base, nvalid, tid);
    float4 rd[2], re[2], rs[2], rr[2];
    fetch32<false>(rd, delta + base, nvalid, tid);
    fetch32<false>(re, Ec + tile, kC, tid);
    fetch32<false>(rs, ScT + tile, kC, tid);
    fetch32<false>(rr, RcT + tile, kC, tid);
    commit16_t<T>(QsT, rq, tid);
    commit16_t<T>(KsT, rk, tid);
    commit16<T, false>(Gs, rg, tid);
    commit32(Ds, rd, tid);
    commit32(Es, re, tid);
    commit32(SsT, rs, tid);
    commit32(RsT, rr, tid);
  }
  __syncthreads();
  float acc[kNT][4], acc2[kNT][4], acck[kNT][4];
  // X1 = strict_lower(dO Dl^T), kept in both orientations
  zero(acc);
  gemm64(acc, Gs, Ds, m0, n0, g, tq);
  mask_tri<true>(acc, m0, n0, g, tq);
  store_acc(X1s, acc, m0, n0, g, tq);
  store_acc_t(X1sT, acc, m0, n0, g, tq);
  // Y = strict_upper(X2) + strict_lower(X2^T), X2 = Dl E^T: every thread writes its elements above
  // the diagonal to both mirror positions and zeroes the diagonal
  zero(acc);
  gemm64(acc, Ds, Es, m0, n0, g, tq);
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = m0 + g + 8 * (e >> 1), cc = n0 + 8 * nt + 2 * tq + (e & 1);
      const float v = round_tf32(acc[nt][e]);
      if (cc > r) {
        Ys[r * kLdV + cc] = v;
        Ys[cc * kLdV + r] = v;
      } else if (cc == r) {
        Ys[r * kLdV + cc] = 0.f;
      }
    }
  }
  // d_query = dO S0 + X1 K ;  d_key = Dl R_end + X1^T Q - Y K - E S0
  zero(acc);
  gemm64(acc, Gs, SsT, m0, n0, g, tq);
  zero(acc2);
  gemm64(acc2, Es, SsT, m0, n0, g, tq);
  zero(acck);
  gemm64(acck, Ds, RsT, m0, n0, g, tq);
  __syncthreads();                 // X1, X1^T, Y tiles complete
  gemm64(acc, X1s, KsT, m0, n0, g, tq);
  gemm64(acck, X1sT, QsT, m0, n0, g, tq);
  gemm64(acc2, Ys, KsT, m0, n0, g, tq);
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

constexpr size_t kTileBytes = (size_t)kC * kLd * sizeof(float);     // prep kernel tiles
constexpr size_t kTileVBytes = (size_t)kC * kLdV * sizeof(float);   // tiles of the chunk kernels
constexpr size_t kPrepTile = kTileBytes;

inline size_t wu_floats(int64_t B, int64_t nc) { return (size_t)B * nc * kC * kDim; }
inline size_t u_floats(int64_t B, int64_t nc) { return (size_t)B * nc * kC * kLdU; }   // U, Ub: padded rows

}  // namespace

// dfw_chunk_umma.cu: the forward chunk walk on the tcgen05 tensor core
int dfw_chunk_forward_umma(const void *q, const void *k, const void *state, const float *W, const float *U,
                           void *out, void *final_state, void *delta, int64_t B, int64_t T_, int dtype,
                           cudaStream_t st);
int dfw_chunk_bwd_seq_umma(const void *go, const void *gs, const void *q, const void *k, const void *delta,
                           const void *final_state, const float *Wb, const float *Ub, float *ScT, float *RcT,
                           float *Ec, void *dv, void *ds, int64_t B, int64_t T_, int dtype, cudaStream_t st);
int dfw_chunk_bwd_par_umma(const void *go, const void *q, const void *k, const void *delta, const float *ScT,
                           const float *RcT, const float *Ec, void *dq, void *dk, int64_t B, int64_t T_, int dtype,
                           cudaStream_t st);
static bool dfw_umma_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("T2FW_DISABLE_DFW_UMMA");
    return !(e && e[0] == '1');
  }();
  return on;
}

bool dfw_chunk_supported(int64_t D, int64_t M, int dtype) {
  return D == kDim && M == kDim && (dtype == T2FW_F16 || dtype == T2FW_BF16);
}

// fp32 [B][n_chunks][64][64] arrays: W and U (forward); Wb, Ub and the per-chunk S0, R_end, E (backward);
// U and Ub with rows of kLdU floats
size_t dfw_chunk_scratch_bytes(int64_t B, int64_t T_, bool backward) {
  const int64_t nc = ceil_div64(T_, kC);
  return align_up(((backward ? 4 : 1) * wu_floats(B, nc) + u_floats(B, nc)) * sizeof(float), 256);
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
  if (dfw_umma_enabled()) {
    const int rc = dfw_chunk_forward_umma(q, k, state, W, U, out, final_state, delta, B, T_,
                                          std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
    if (rc != T2FW_ERR_UNSUPPORTED) return rc;
  }
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(7 * kTileVBytes)));
  dfw_chunk_fwd_kernel<T><<<(unsigned)B, kSeqThreads, 7 * kTileVBytes, st>>>(
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
  float *Sc = Ub + u_floats(B, nc), *Rc = Sc + wu_floats(B, nc), *Ec = Rc + wu_floats(B, nc);
  int seq_rc = T2FW_ERR_UNSUPPORTED;
  if (dfw_umma_enabled())
    seq_rc = dfw_chunk_bwd_seq_umma(go, gs, q, k, delta, final_state, Wb, Ub, Sc, Rc, Ec, dv, ds, B, T_,
                                    std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
  if (seq_rc != T2FW_OK && seq_rc != T2FW_ERR_UNSUPPORTED) return seq_rc;
  if (seq_rc == T2FW_ERR_UNSUPPORTED) {
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_bwd_seq_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(7 * kTileVBytes)));
    dfw_chunk_bwd_seq_kernel<T><<<(unsigned)B, kSeqThreads, 7 * kTileVBytes, st>>>(
        (const T *)go, (const T *)gs, (const T *)q, (const T *)k, (const float *)delta, (const T *)final_state,
        Wb, Ub, Sc, Rc, Ec, (T *)dv, (T *)ds, T_, nc);
  }
  int par_rc = T2FW_ERR_UNSUPPORTED;
  if (dfw_umma_enabled())
    par_rc = dfw_chunk_bwd_par_umma(go, q, k, delta, Sc, Rc, Ec, dq, dk, B, T_,
                                    std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
  if (par_rc != T2FW_OK && par_rc != T2FW_ERR_UNSUPPORTED) return par_rc;
  if (par_rc == T2FW_ERR_UNSUPPORTED) {
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_bwd_par_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(10 * kTileVBytes)));
    dfw_chunk_bwd_par_kernel<T><<<(unsigned)(B * nc), kSeqThreads, 10 * kTileVBytes, st>>>(
        (const T *)go, (const T *)q, (const T *)k, (const float *)delta, Sc, Rc, Ec, (T *)dq, (T *)dk, T_, nc);
  }
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
