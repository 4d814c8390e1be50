// Chunked decay-rule forward for D = K = 64, 16-bit storage (see lfw_chunk.cuh for the algebra).
//
// Replaces the reference's sequential scan + output einsum (t2fw/csrc/lfw_kernel.cu:18-59,
// t2fw/csrc/lfw.cpp:45) with three launches:
//   1. lfw_chunk_local_kernel  (b, chunk) in parallel: the chunk's own contribution to the
//      state, L_c, and the chunk's total decay vectors (fp32 scratch)
//   2. lfw_chunk_carry_kernel  elementwise scan over chunks: start-of-chunk states (fp32,
//      in place over L_c) and the 16-bit checkpoints, slot c = state after chunk c
//   3. lfw_chunk_output_kernel (b, chunk) in parallel: outputs of the chunk from its start
//      state, state carried through the four sub-blocks in fp32 accumulators
// Scratch layout (floats): L[B][nc][64][64] | Ac[B][nc][64] | Gc[B][nc][64] | flags[B][nc] (int)
// | rowflag[B] (int).  flags mark chunks whose gate products left the safe range; such batch
// rows are recomputed by the scan kernels afterwards.
#include <cstdlib>
#include <type_traits>

#include "lfw_chunk.cuh"

namespace t2fw {

using namespace chunk;

// persistent, prefetching version of the output phase (lfw_chunk_fwd_out.cu)
int lfw_chunk_output_persist(const void *x, const void *f, const void *q, const void *k, const void *fk,
                             const float *Sstart, void *out, int64_t B, int64_t T_, int dtype,
                             cudaStream_t st);
// tcgen05 output phase on 64-step chunks (lfw_c64_fwd.cu)
int lfw_c64_forward_out(const void *x, const void *f, const void *q, const void *k, const void *fk,
                        const float *Sstart, void *out, int *rowflag, int64_t B, int64_t T_, int dtype,
                        cudaStream_t st);
static bool c64_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("T2FW_DISABLE_C64");
    return !(e && e[0] == '1');
  }();
  return on && umma_enabled();
}
static bool persist_enabled() {
  const char *e = std::getenv("T2FW_DISABLE_PERSIST");
  return !(e && e[0] == '1');
}

namespace {

struct FwdScratch {
  float *L, *Ac, *Gc;
  int *flags, *rowflag;
};

__host__ __device__ inline size_t fwd_scratch_floats(int64_t B, int64_t nc) {
  return (size_t)B * nc * kDim * kDim + 2 * (size_t)B * nc * kDim + (size_t)B * nc + (size_t)B;
}

inline FwdScratch carve(void *scratch, int64_t B, int64_t nc) {
  FwdScratch s;
  s.L = static_cast<float *>(scratch);
  s.Ac = s.L + (size_t)B * nc * kDim * kDim;
  s.Gc = s.Ac + (size_t)B * nc * kDim;
  s.flags = reinterpret_cast<int *>(s.Gc + (size_t)B * nc * kDim);
  s.rowflag = s.flags + (size_t)B * nc;
  return s;
}

// state <- (aI gI^T) .* state ; state += (Xt*aI)^T (Kt*gI) for sub-block I; warp w owns rows 16w..
__device__ __forceinline__ void state_step(float (&S)[8][4], const float *Xt, const float *Kt,
                                           const float *aI, const float *gI, int I, int w, int g,
                                           int tq, bool scale_old) {
  const float a_lo = aI[I * kDim + 16 * w + g], a_hi = aI[I * kDim + 16 * w + g + 8];
  if (scale_old) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float2 gg = *reinterpret_cast<const float2 *>(gI + I * kDim + nt * 8 + 2 * tq);
      S[nt][0] *= a_lo * gg.x;
      S[nt][1] *= a_lo * gg.y;
      S[nt][2] *= a_hi * gg.x;
      S[nt][3] *= a_hi * gg.y;
    }
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

template <typename T>
__global__ void __launch_bounds__(kThreads)
lfw_chunk_local_kernel(const T *__restrict__ x, const T *__restrict__ f, const T *__restrict__ k,
                       const T *__restrict__ fk, float *__restrict__ L, float *__restrict__ Ac,
                       float *__restrict__ Gc, int *__restrict__ flags, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Xt = sm, *Kt = Xt + kC * kLd, *aI = Kt + kC * kLd, *gI = aI + kNSub * kDim;
  __shared__ int s_flag;
  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc;
  const int64_t t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  if (threadIdx.x == 0) s_flag = 0;
  __syncthreads();
  const size_t base = ((size_t)b * T_ + t0) * kDim;
  bool bad = prep_side<T>(fk + base, nullptr, k + base, nvalid, nullptr, Kt, nullptr, nullptr, gI);
  bad |= prep_side<T>(f + base, nullptr, x + base, nvalid, nullptr, Xt, nullptr, nullptr, aI);
  if (bad) s_flag = 1;
  __syncthreads();

  float S[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
#pragma unroll
  for (int I = 0; I < kNSub; ++I) state_step(S, Xt, Kt, aI, gI, I, w, g, tq, I > 0);

  float *Lc = L + ((size_t)b * nc + c) * kDim * kDim;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<float2 *>(Lc + (16 * w + g) * kDim + nt * 8 + 2 * tq) = make_float2(S[nt][0], S[nt][1]);
    *reinterpret_cast<float2 *>(Lc + (16 * w + g + 8) * kDim + nt * 8 + 2 * tq) = make_float2(S[nt][2], S[nt][3]);
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

// One thread per (b, d, 4 consecutive k): S_{c+1} = (Ac Gc^T) S_c + L_c.  L_c is overwritten with
// the state at the START of chunk c; ckpt slot c receives the state after chunk c.
template <typename T>
__global__ void __launch_bounds__(128, 6)
lfw_chunk_carry_kernel(const T *__restrict__ state, float *__restrict__ L, const float *__restrict__ Ac,
                       const float *__restrict__ Gc, const int *__restrict__ flags,
                       int *__restrict__ rowflag, T *__restrict__ ckpt, int64_t B, int64_t nc) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * kDim * (kDim / 4)) return;
  const int64_t b = idx / (kDim * (kDim / 4));
  const int d = (int)((idx / (kDim / 4)) % kDim);
  const int k0 = (int)(idx % (kDim / 4)) * 4;
  const T *sp = state + ((size_t)b * kDim + d) * kDim + k0;
  float2 s01 = Pair<T>::ld(sp), s23 = Pair<T>::ld(sp + 2);
  float S[4] = {s01.x, s01.y, s23.x, s23.y};
  int any = 0;
  // batches of 8 chunks: all loads of a batch are issued before its dependent FMA chain
  for (int64_t c0 = 0; c0 < nc; c0 += 8) {
    float4 l[8], gg[8];
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t c = (c0 + j < nc) ? c0 + j : nc - 1;
      const size_t bc = (size_t)b * nc + c;
      l[j] = *reinterpret_cast<const float4 *>(L + (bc * kDim + d) * kDim + k0);
      a[j] = Ac[bc * kDim + d];
      gg[j] = *reinterpret_cast<const float4 *>(Gc + bc * kDim + k0);
      if (d == 0 && k0 == 0) any |= flags[bc];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (c0 + j < nc) {
        const size_t bc = (size_t)b * nc + c0 + j;
        *reinterpret_cast<float4 *>(L + (bc * kDim + d) * kDim + k0) = make_float4(S[0], S[1], S[2], S[3]);
        S[0] = a[j] * gg[j].x * S[0] + l[j].x;
        S[1] = a[j] * gg[j].y * S[1] + l[j].y;
        S[2] = a[j] * gg[j].z * S[2] + l[j].z;
        S[3] = a[j] * gg[j].w * S[3] + l[j].w;
        T *cp = ckpt + (bc * kDim + d) * kDim + k0;
        Pair<T>::st(cp, S[0], S[1]);
        Pair<T>::st(cp + 2, S[2], S[3]);
      }
    }
  }
  if (d == 0 && k0 == 0) rowflag[b] = any;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
lfw_chunk_output_kernel(const T *__restrict__ x, const T *__restrict__ f, const T *__restrict__ q,
                        const T *__restrict__ k, const T *__restrict__ fk,
                        const float *__restrict__ Sstart, T *__restrict__ out, int64_t T_, int64_t nc) {
  extern __shared__ __align__(16) float sm[];
  float *Qt = sm, *Kt = Qt + kC * kLd, *Xt = Kt + kC * kLd, *Ap = Xt + kC * kLd;
  float *P = Ap + kC * kLd;                     // [4][16][kLdP]
  float *aI = P + kNSub * kSub * kLdP, *gI = aI + kNSub * kDim;
  const int64_t b = blockIdx.x / nc, c = blockIdx.x % nc;
  const int64_t t0 = c * kC;
  const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const size_t base = ((size_t)b * T_ + t0) * kDim;
  prep_side<T>(fk + base, q + base, k + base, nvalid, Qt, Kt, nullptr, nullptr, gI);
  prep_side<T>(f + base, nullptr, x + base, nvalid, nullptr, Xt, Ap, nullptr, aI);
  __syncthreads();

  // Pair tile of sub-block w: P[t][i] = Qt_t . Kt_i for i <= t, else 0.
  {
    float acc[2][4] = {};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t a[4];
      lda(a, Qt, kLd, 16 * w, 8 * ks, g, tq);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        uint32_t bb[2];
        ldb_t(bb, Kt, kLd, 8 * ks, 16 * w + 8 * nt, g, tq);
        mma_tf32(acc[nt], a, bb);
      }
    }
    float *Pw = P + w * kSub * kLdP;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int i0 = 8 * nt + 2 * tq;
      Pw[g * kLdP + i0] = (i0 <= g) ? round_tf32(acc[nt][0]) : 0.f;
      Pw[g * kLdP + i0 + 1] = (i0 + 1 <= g) ? round_tf32(acc[nt][1]) : 0.f;
      Pw[(g + 8) * kLdP + i0] = (i0 <= g + 8) ? round_tf32(acc[nt][2]) : 0.f;
      Pw[(g + 8) * kLdP + i0 + 1] = (i0 + 1 <= g + 8) ? round_tf32(acc[nt][3]) : 0.f;
    }
  }

  // start-of-chunk state, rows 16w+g / +8, columns nt*8 + 2tq, +1
  float S[8][4];
  const float *Sc = Sstart + ((size_t)b * nc + c) * kDim * kDim;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const float2 lo = *reinterpret_cast<const float2 *>(Sc + (16 * w + g) * kDim + nt * 8 + 2 * tq);
    const float2 hi = *reinterpret_cast<const float2 *>(Sc + (16 * w + g + 8) * kDim + nt * 8 + 2 * tq);
    S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
  }
  __syncthreads();   // P complete

  T *ob = out + base;
#pragma unroll 1
  for (int I = 0; I < kNSub; ++I) {
    // O^T[d][t] for d in the warp's 16 rows, t in sub-block I
    float O[2][4] = {};
#pragma unroll
    for (int nk = 0; nk < 8; ++nk) {
      // A = state (accumulator registers reused as operand): contraction index kk<4 -> column
      // 2kk of the 8-column group, kk>=4 -> column 2(kk-4)+1; B is read with the same mapping.
      uint32_t a[4] = {to_tf32(S[nk][0]), to_tf32(S[nk][2]), to_tf32(S[nk][1]), to_tf32(S[nk][3])};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float2 qv = *reinterpret_cast<const float2 *>(Qt + (I * kSub + 8 * nt + g) * kLd + nk * 8 + 2 * tq);
        uint32_t bb[2] = {__float_as_uint(qv.x), __float_as_uint(qv.y)};
        mma_tf32(O[nt], a, bb);
      }
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t a[4];
      lda_t(a, Xt, kLd, 16 * w, I * kSub + 8 * ks, g, tq);      // A[d][i] = Xt[i][d]
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        uint32_t bb[2];
        ldb_t(bb, P + I * kSub * kLdP, kLdP, 8 * ks, 8 * nt, g, tq);   // B[i][t] = P[t][i]
        mma_tf32(O[nt], a, bb);
      }
    }
    // out[t][d] = ap[t][d] * O^T[d][t]
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = I * kSub + 8 * nt + 2 * tq + (e & 1);
        const int d = 16 * w + g + ((e & 2) ? 8 : 0);
        if (t < nvalid) Elem<T>::st(ob + (size_t)t * kDim + d, Ap[t * kLd + d] * O[nt][e]);
      }
    }
    if (I + 1 < kNSub) state_step(S, Xt, Kt, aI, gI, I, w, g, tq, true);
  }
}

}  // namespace

bool lfw_chunk_supported(int64_t D, int64_t K, int dtype, int64_t ckpt_every) {
  return D == kDim && K == kDim && ckpt_every == kC && (dtype == T2FW_F16 || dtype == T2FW_BF16);
}

size_t lfw_chunk_forward_scratch_bytes(int64_t B, int64_t T_) {
  const int64_t nc = ceil_div64(T_, kC);
  return align_up(fwd_scratch_floats(B, nc) * sizeof(float), 256);
}

template <typename T>
static int chunk_forward_typed(const void *x, const void *f, const void *q, const void *k,
                               const void *fk, const void *state, void *out, void *ckpt, int64_t B,
                               int64_t T_, void *scratch, cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC);
  FwdScratch s = carve(scratch, B, nc);
  const size_t sm_local = (2 * kC * kLd + 2 * kNSub * kDim) * sizeof(float);
  const size_t sm_out = (4 * kC * kLd + kNSub * kSub * kLdP + 2 * kNSub * kDim) * sizeof(float);
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_chunk_output_kernel<T>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_out));
  bool local_done = false;
  if (umma_enabled()) {
    const int rc = lfw_chunk_local_umma(false, x, f, k, fk, s.L, s.Ac, s.Gc, s.flags, B, T_,
                                        std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
    if (rc == T2FW_OK) local_done = true;
    else if (rc != T2FW_ERR_UNSUPPORTED) return rc;
  }
  if (!local_done) {
    lfw_chunk_local_kernel<T><<<(unsigned)(B * nc), kThreads, sm_local, st>>>(
        (const T *)x, (const T *)f, (const T *)k, (const T *)fk, s.L, s.Ac, s.Gc, s.flags, T_, nc);
    T2FW_CHECK_LAUNCH(1);
  }
  const int64_t n_carry = B * kDim * (kDim / 4);
  lfw_chunk_carry_kernel<T><<<(unsigned)ceil_div64(n_carry, 128), 128, 0, st>>>(
      (const T *)state, s.L, s.Ac, s.Gc, s.flags, s.rowflag, (T *)ckpt, B, nc);
  T2FW_CHECK_LAUNCH(1);
  int rc_out = T2FW_ERR_UNSUPPORTED;
  if (c64_enabled())
    rc_out = lfw_c64_forward_out(x, f, q, k, fk, s.L, out, s.rowflag, B, T_,
                                 std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
  if (rc_out == T2FW_ERR_UNSUPPORTED && persist_enabled())
    rc_out = lfw_chunk_output_persist(x, f, q, k, fk, s.L, out, B, T_,
                                      std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
  if (rc_out == T2FW_ERR_UNSUPPORTED) {
    lfw_chunk_output_kernel<T><<<(unsigned)(B * nc), kThreads, sm_out, st>>>(
        (const T *)x, (const T *)f, (const T *)q, (const T *)k, (const T *)fk, s.L, (T *)out, T_, nc);
    T2FW_CHECK_LAUNCH(1);
    rc_out = T2FW_OK;
  }
  return rc_out;
}

int lfw_chunk_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                      const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int dtype,
                      void *scratch, cudaStream_t st, const int **rowflag_out) {
  const int64_t nc = ceil_div64(T_, kC);
  if (rowflag_out) *rowflag_out = carve(scratch, B, nc).rowflag;
  if (dtype == T2FW_F16)
    return chunk_forward_typed<__half>(x, f, q, k, fk, state, out, ckpt, B, T_, scratch, st);
  return chunk_forward_typed<__nv_bfloat16>(x, f, q, k, fk, state, out, ckpt, B, T_, scratch, st);
}

}  // namespace t2fw
