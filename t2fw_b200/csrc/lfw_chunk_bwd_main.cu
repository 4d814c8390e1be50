// Main kernel of the chunked decay-rule backward (D = K = 64, 16-bit storage): one CTA per
// (batch row, 64-step chunk), eight warps specialised by side.
//
//   warps 0-3 ("k side"): own the forward state.  They prepare the k-side operands (Qt, Kt,
//       prefixes gp), the pair tile P, recompute the state at the start of each of the four
//       sub-blocks from the chunk's checkpoint once (kept in shared memory), and per sub-block
//       produce d_q, d_k, d_f_key for a 16-column slice each.
//   warps 4-7 ("d side"): own the state gradient R (fp32 accumulators).  They prepare the d-side
//       operands (dOt, Xt, prefixes ap), the pair tile Z, and per sub-block produce d_x, d_f for
//       a 16-column slice each, then step R back across the sub-block.
//
// Per sub-block (start state S0, end gradient R, block decays aI, gI):
//   dq = gp .* (dOt S0 + Z Kt)                      dk = (Z^T Qt + gI .* ((Xt aI) R)) ./ gp
//   dx = (P^T dOt + aI .* ((Kt gI) R^T)) ./ ap      R_prev = (aI gI^T) .* R + dOt^T Qt
//   H  = suffix_t[Qt.*(dOt S0 + Z Kt) - Kt.*(Z^T Qt)] + exclusive_prefix_t[Kt.*gI.*((Xt aI) R)]
//        + gI .* sum_d aI R S0 ;     d_f_key = H ./ g      (d side: the same with roles exchanged)
// The only cancelling part of H (the in-block pair terms) is built from identical TF32-rounded
// operands on both sides; gates smaller than 2^-10 get the exact, cancellation-free formula.
#include "lfw_chunk.cuh"

namespace t2fw {

using namespace chunk;

namespace {

constexpr int kMainThreads = 256;
constexpr int kStgLd = kDim + 8;   // row stride (elements) of the 16-bit output staging tiles
constexpr int kFixCap = 256;       // tiny-gate elements per sub-block that get the exact formula
constexpr float kTinyGate = 9.765625e-4f;   // 2^-10

constexpr size_t main_smem_bytes(size_t elt) {
  return (size_t)(11 * kC * kLd + 2 * kNSub * kSub * kLdP + 2 * kNSub * kDim + 2 * kDim + kFixCap) *
             sizeof(float) + 5 * kSub * kStgLd * elt;
}

// publish an accumulator-layout register tile (rows 16w+g / +8, cols nt*8+2tq, +1) as TF32 values
__device__ __forceinline__ void publish_tile(float *tile, const float (&S)[8][4], int w, int g, int tq) {
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<float2 *>(tile + (16 * w + g) * kLd + nt * 8 + 2 * tq) =
        make_float2(round_tf32(S[nt][0]), round_tf32(S[nt][1]));
    *reinterpret_cast<float2 *>(tile + (16 * w + g + 8) * kLd + nt * 8 + 2 * tq) =
        make_float2(round_tf32(S[nt][2]), round_tf32(S[nt][3]));
  }
}

template <typename T>
__global__ void __launch_bounds__(kMainThreads, 1)
lfw_chunk_bwd_main_kernel(const T *__restrict__ go, const T *__restrict__ x, const T *__restrict__ f,
                          const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ fk,
                          const T *__restrict__ state, const T *__restrict__ ckpt,
                          const float *__restrict__ Rend, T *__restrict__ dx, T *__restrict__ df,
                          T *__restrict__ dq, T *__restrict__ dk, T *__restrict__ dfk,
                          int *__restrict__ rowflag, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Qt = sm, *Kt = Qt + kC * kLd, *Xt = Kt + kC * kLd, *dOt = Xt + kC * kLd;
  float *Gp = dOt + kC * kLd, *Ap = Gp + kC * kLd;
  float *Sst = Ap + kC * kLd;                        // [4] states at the start of sub-blocks 0..3
  float *Rm = Sst + kNSub * kDim * kLd;              // state gradient at the end of the sub-block
  float *Pr = Rm + kDim * kLd, *Zr = Pr + kNSub * kSub * kLdP;
  float *aI = Zr + kNSub * kSub * kLdP, *gI = aI + kNSub * kDim;
  float *c4k = gI + kNSub * kDim, *c4d = c4k + kDim;
  int *fix_list = reinterpret_cast<int *>(c4d + kDim);
  T *stg = reinterpret_cast<T *>(fix_list + kFixCap);   // dq, dk, dfk, dx, df tiles [16][kStgLd]
  __shared__ int fix_n;

  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc;
  const int64_t t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const bool kgroup = threadIdx.x < 128;             // warps 0-3: k side, warps 4-7: d side
  const int tid = threadIdx.x & 127;
  const int w = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const size_t base = ((size_t)b * T_ + t0) * kDim;

  if (threadIdx.x == 0) fix_n = 0;
  if (kgroup)
    prep_side<T>(fk + base, q + base, k + base, nvalid, Qt, Kt, Gp, nullptr, gI, tid);
  else
    prep_side<T>(f + base, go + base, x + base, nvalid, dOt, Xt, Ap, nullptr, aI, tid);
  __syncthreads();

  // pair tile of sub-block w: P = tril(Qt Kt^T) (k group), Z = tril(dOt Xt^T) (d group)
  {
    const float *Am = kgroup ? Qt : dOt, *Bm = kgroup ? Kt : Xt;
    float acc[2][4] = {};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t a[4];
      lda(a, Am, kLd, 16 * w, 8 * ks, g, tq);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        uint32_t bb[2];
        ldb_t(bb, Bm, kLd, 8 * ks, 16 * w + 8 * nt, g, tq);
        mma_tf32(acc[nt], a, bb);
      }
    }
    float *Pw = (kgroup ? Pr : Zr) + w * kSub * kLdP;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int i0 = 8 * nt + 2 * tq;
      Pw[g * kLdP + i0] = (i0 <= g) ? round_tf32(acc[nt][0]) : 0.f;
      Pw[g * kLdP + i0 + 1] = (i0 + 1 <= g) ? round_tf32(acc[nt][1]) : 0.f;
      Pw[(g + 8) * kLdP + i0] = (i0 <= g + 8) ? round_tf32(acc[nt][2]) : 0.f;
      Pw[(g + 8) * kLdP + i0 + 1] = (i0 + 1 <= g + 8) ? round_tf32(acc[nt][3]) : 0.f;
    }
  }

  float R[8][4];   // d group: state gradient, rows 16w+g / +8, columns nt*8 + 2tq, +1
  if (kgroup) {
    // forward states at the start of the four sub-blocks, from the chunk's checkpoint
    const T *Sc = (c == 0) ? state + (size_t)b * kDim * kDim
                           : ckpt + ((size_t)b * nc + (c - 1)) * kDim * kDim;
    float S[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float2 lo = Pair<T>::ld(Sc + (16 * w + g) * kDim + nt * 8 + 2 * tq);
      const float2 hi = Pair<T>::ld(Sc + (16 * w + g + 8) * kDim + nt * 8 + 2 * tq);
      S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
    }
    publish_tile(Sst, S, w, g, tq);
#pragma unroll 1
    for (int J = 0; J + 1 < kNSub; ++J) {
      state_step_regs(S, Xt, Kt, aI, gI, J, w, g, tq);
      publish_tile(Sst + (J + 1) * kDim * kLd, S, w, g, tq);
    }
  } else {
    const float *Rc = Rend + ((size_t)b * nc + c) * kDim * kDim;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float2 lo = *reinterpret_cast<const float2 *>(Rc + (16 * w + g) * kDim + nt * 8 + 2 * tq);
      const float2 hi = *reinterpret_cast<const float2 *>(Rc + (16 * w + g + 8) * kDim + nt * 8 + 2 * tq);
      R[nt][0] = lo.x; R[nt][1] = lo.y; R[nt][2] = hi.x; R[nt][3] = hi.y;
    }
    publish_tile(Rm, R, w, g, tq);
  }
  __syncthreads();

  const int n0 = 16 * w;            // this warp's 16-column slice (k columns or d columns)
#pragma unroll 1
  for (int I = kNSub - 1; I >= 0; --I) {
    const float *S0 = Sst + I * kDim * kLd;
    const float *PI = Pr + I * kSub * kLdP, *ZI = Zr + I * kSub * kLdP;
    const float *aIb = aI + I * kDim, *gIb = gI + I * kDim;
    const int r0 = I * kSub;

    // boundary term of the slice: sum over the other axis of decay .* R .* S0
    {
      const int cl = lane & 15, half = lane >> 4;
      float s = 0.f;
      if (kgroup) {
        const int col = n0 + cl;                 // k column; sum over 32 d rows
#pragma unroll 8
        for (int d = 32 * half; d < 32 * half + 32; ++d) s += aIb[d] * Rm[d * kLd + col] * S0[d * kLd + col];
        s += __shfl_xor_sync(0xffffffffu, s, 16);
        if (half == 0) c4k[col] = gIb[col] * s;
      } else {
        const int row = n0 + cl;                 // d row; sum over 32 k columns
#pragma unroll 8
        for (int kk = 32 * half; kk < 32 * half + 32; ++kk) s += gIb[kk] * Rm[row * kLd + kk] * S0[row * kLd + kk];
        s += __shfl_xor_sync(0xffffffffu, s, 16);
        if (half == 0) c4d[row] = aIb[row] * s;
      }
      __syncwarp();
    }

    if (kgroup) {
      // ================= k side: d_q, d_k, d_f_key for columns n0..n0+15 ====================
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
        for (int e = 0; e < 2; ++e) {
          const int col = n0 + 8 * nt + 2 * tq + e;
          const float gIk = gIb[col], c4 = c4k[col];
          float v[2], b3[2], rg[2], gprev[2], dqv[2], dkv[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
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
    } else {
      // ================= d side: d_x, d_f for columns n0..n0+15 ==============================
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
      // state gradient at the start of the sub-block (registers only)
      grad_step_regs(R, dOt, Qt, aI, gI, I, w, g, tq, true);
    }
    __syncthreads();   // staging and the tiny-gate list are complete; Rm still holds the old R

    // ---- exact gate gradients where the gate is too small for the cancelling form ----------
    //   dg_t[k] = (1/g_t) sum_d M[d] N[d],  M = S0[:,k] + sum_{i<t} Xt_i Kt_i[k],
    //                                       N = aI gI[k] R[:,k] + sum_{s>=t} dOt_s Qt_s[k]
    // (every term of N carries the factor g_t, so nothing cancels); d side with d and k exchanged.
    if (fix_n > 0) {
      const int n_fix = fix_n < kFixCap ? fix_n : kFixCap;
      if (fix_n > kFixCap && threadIdx.x == 0) atomicExch(rowflag + b, 1);   // the scan kernels redo the row
      for (int e = threadIdx.x >> 5; e < n_fix; e += kMainThreads / 32) {
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

    // ---- coalesced write of the five 16 x 64 result tiles; publish R for the next sub-block --
    {
      T *dst[5] = {dq, dk, dfk, dx, df};
      for (int idx = threadIdx.x; idx < 5 * kSub * 8; idx += kMainThreads) {
        const int it = idx >> 7, r = (idx >> 3) & 15, ch = idx & 7;
        if (r0 + r < nvalid) {
          const uint4 val = *reinterpret_cast<const uint4 *>(stg + (it * kSub + r) * kStgLd + ch * 8);
          *reinterpret_cast<uint4 *>(dst[it] + base + (size_t)(r0 + r) * kDim + ch * 8) = val;
        }
      }
      if (!kgroup && I > 0) publish_tile(Rm, R, w, g, tq);
      if (threadIdx.x == 0) fix_n = 0;
    }
    __syncthreads();   // R published, staging free, counter reset
  }
}

}  // namespace

int lfw_chunk_bwd_main(const void *go, const void *x, const void *f, const void *q, const void *k,
                       const void *fk, const void *state, const void *ckpt, const float *Rend,
                       void *dx, void *df, void *dq, void *dk, void *dfk, int *rowflag, int64_t B,
                       int64_t T_, int dtype, cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC);
  const size_t smem = main_smem_bytes(2);
  const unsigned grid = (unsigned)(B * nc);
#define T2FW_LAUNCH(TT)                                                                               \
  do {                                                                                                \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_chunk_bwd_main_kernel<TT>,                               \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
    lfw_chunk_bwd_main_kernel<TT><<<grid, kMainThreads, smem, st>>>(                                  \
        (const TT *)go, (const TT *)x, (const TT *)f, (const TT *)q, (const TT *)k, (const TT *)fk,   \
        (const TT *)state, (const TT *)ckpt, Rend, (TT *)dx, (TT *)df, (TT *)dq, (TT *)dk, (TT *)dfk, \
        rowflag, T_, nc);                                                                             \
  } while (0)
  if (dtype == T2FW_F16) T2FW_LAUNCH(__half); else T2FW_LAUNCH(__nv_bfloat16);
#undef T2FW_LAUNCH
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw
