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
#include <cstdlib>
#include <type_traits>

#include "lfw_chunk.cuh"

namespace t2fw {

using namespace chunk;

// main kernel (lfw_chunk_bwd_main.cu)
int lfw_chunk_bwd_main(const void *go, const void *x, const void *f, const void *q, const void *k,
                       const void *fk, const void *state, const void *ckpt, const float *Rend,
                       void *dx, void *df, void *dq, void *dk, void *dfk, int *rowflag, int64_t B,
                       int64_t T_, int dtype, cudaStream_t st);

// tcgen05 main kernel (lfw_chunk_bwd_umma.cu); T2FW_ERR_UNSUPPORTED without a launch if it cannot run
int lfw_chunk_bwd_main_umma(const void *go, const void *x, const void *f, const void *q, const void *k,
                            const void *fk, const void *state, const void *ckpt, const float *Rend,
                            void *dx, void *df, void *dq, void *dk, void *dfk, int *rowflag, int64_t B,
                            int64_t T_, int dtype, cudaStream_t st);

// tcgen05 main kernel on 64-step chunks (lfw_c64_bwd.cu)
int lfw_c64_backward_main(const void *go, const void *x, const void *f, const void *q, const void *k,
                          const void *fk, const void *state, const void *ckpt, const float *Rend, void *dx,
                          void *df, void *dq, void *dk, void *dfk, int *rowflag, int64_t B, int64_t T_,
                          int dtype, cudaStream_t st);

namespace {

bool c64_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("T2FW_DISABLE_C64");
    return !(e && e[0] == '1');
  }();
  return on && umma_enabled();
}

bool bwd_umma_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("T2FW_DISABLE_BWD_UMMA");
    return !(e && e[0] == '1');
  }();
  return on && umma_enabled();
}

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
  for (int I = kNSub - 1; I >= 0; --I) grad_step_regs(R, dOt, Qt, aI, gI, I, w, g, tq, I < kNSub - 1);

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
__global__ void __launch_bounds__(128, 6)
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
  bool local_done = false;
  if (umma_enabled()) {
    const int rc = lfw_chunk_local_umma(true, go, f, q, fk, s.G, s.Ac, s.Gc, s.flags, B, T_,
                                        std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16, st);
    if (rc == T2FW_OK) local_done = true;
    else if (rc != T2FW_ERR_UNSUPPORTED) return rc;
  }
  if (!local_done) {
    lfw_chunk_bwd_local_kernel<T><<<(unsigned)(B * nc), kThreads, sm_local, st>>>(
        (const T *)go, (const T *)f, (const T *)q, (const T *)fk, s.G, s.Ac, s.Gc, s.flags, T_, nc);
    T2FW_CHECK_LAUNCH(1);
  }
  const int64_t n_carry = B * kDim * (kDim / 4);
  lfw_chunk_bwd_carry_kernel<T><<<(unsigned)ceil_div64(n_carry, 128), 128, 0, st>>>(
      (const T *)gs, s.G, s.Ac, s.Gc, s.flags, s.rowflag, (T *)ds, B, nc);
  T2FW_CHECK_LAUNCH(1);
  const int dt = std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16;
  if (c64_enabled()) {
    const int rc = lfw_c64_backward_main(go, x, f, q, k, fk, state, ckpt, s.G, dx, df, dq, dk, dfk,
                                         s.rowflag, B, T_, dt, st);
    if (rc != T2FW_ERR_UNSUPPORTED) return rc;
  }
  if (bwd_umma_enabled()) {
    const int rc = lfw_chunk_bwd_main_umma(go, x, f, q, k, fk, state, ckpt, s.G, dx, df, dq, dk, dfk,
                                           s.rowflag, B, T_, dt, st);
    if (rc != T2FW_ERR_UNSUPPORTED) return rc;
  }
  return lfw_chunk_bwd_main(go, x, f, q, k, fk, state, ckpt, s.G, dx, df, dq, dk, dfk, s.rowflag, B, T_,
                            dt, st);
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
