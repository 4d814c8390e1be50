// Delta-rule ("DFW") scan kernels.
//
//   o_t = S_{t-1} q_t ,  delta_t = v_t - S_{t-1} k_t ,  S_t = S_{t-1} + delta_t k_t^T
//
// Same organisation as the decay-rule scan: a warp owns a few lines of the D x M state in
// registers (accumulation type), the lanes spread along the other axis, time is sequential,
// every reduction is a warp reduction.
//
//   forward  (own = d rows)    : outputs, delta, final state
//                                (reference kernel: t2fw/csrc/dfw_kernel.cu:105-196)
//   backward rows (own = d)    : d_value_t = G_t k_t, the G recurrence, d_state
//                                (reference kernel: t2fw/csrc/dfw_kernel.cu:198-283)
//   backward cols (own = m)    : d_query, d_key; walks the state column backwards from the
//                                final state, S_{t-1} = S_t - delta_t k_t^T
//                                (reference kernel: t2fw/csrc/dfw_kernel.cu:285-384)
#include "common.cuh"

namespace t2fw {

namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kOwn = 2;

template <typename T, int NL>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
dfw_fwd_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
               const T *__restrict__ state, T *__restrict__ out, T *__restrict__ fin,
               typename Elem<T>::acc *__restrict__ delta, int64_t B, int64_t T_, int64_t D,
               int64_t M) {
  using A = typename Elem<T>::acc;
  const int lane = threadIdx.x & 31;
  const int64_t groups = (D + kOwn - 1) / kOwn;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (warp >= B * groups) return;
  const int64_t b = warp / groups;
  const int64_t r0 = (warp % groups) * kOwn;

  A S[kOwn][NL];
#pragma unroll
  for (int o = 0; o < kOwn; ++o)
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t row = r0 + o, c = lane + 32 * j;
      S[o][j] = (row < D && c < M) ? Elem<T>::ld(state + (b * D + row) * M + c) : A(0);
    }
  for (int64_t t = 0; t < T_; ++t) {
    const int64_t bm = (b * T_ + t) * M, bd = (b * T_ + t) * D;
    A kl[NL], ql[NL];
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t c = lane + 32 * j;
      kl[j] = c < M ? Elem<T>::ld(k + bm + c) : A(0);
      ql[j] = c < M ? Elem<T>::ld(q + bm + c) : A(0);
    }
#pragma unroll
    for (int o = 0; o < kOwn; ++o) {
      const int64_t row = r0 + o;
      const bool in = row < D;
      A so = A(0), sk = A(0);
#pragma unroll
      for (int j = 0; j < NL; ++j) {
        so += S[o][j] * ql[j];
        sk += S[o][j] * kl[j];
      }
      so = warp_sum(so);
      sk = warp_sum(sk);
      const A dl = (in ? Elem<T>::ld(v + bd + row) : A(0)) - sk;
#pragma unroll
      for (int j = 0; j < NL; ++j) S[o][j] += dl * kl[j];
      if (lane == 0 && in) {
        Elem<T>::st(out + bd + row, so);
        delta[bd + row] = dl;
      }
    }
  }
#pragma unroll
  for (int o = 0; o < kOwn; ++o)
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t row = r0 + o, c = lane + 32 * j;
      if (row < D && c < M) Elem<T>::st(fin + (b * D + row) * M + c, S[o][j]);
    }
}

// rows: G_t row recurrence, d_value, d_state
template <typename T, int NL>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
dfw_bwd_rows_kernel(const T *__restrict__ go, const T *__restrict__ gs, const T *__restrict__ q,
                    const T *__restrict__ k, T *__restrict__ dv, T *__restrict__ ds,
                    typename Elem<T>::acc *__restrict__ dv_acc, int64_t B, int64_t T_, int64_t D,
                    int64_t M) {
  using A = typename Elem<T>::acc;
  const int lane = threadIdx.x & 31;
  const int64_t groups = (D + kOwn - 1) / kOwn;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (warp >= B * groups) return;
  const int64_t b = warp / groups;
  const int64_t r0 = (warp % groups) * kOwn;

  A G[kOwn][NL];
#pragma unroll
  for (int o = 0; o < kOwn; ++o)
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t row = r0 + o, c = lane + 32 * j;
      G[o][j] = (row < D && c < M) ? Elem<T>::ld(gs + (b * D + row) * M + c) : A(0);
    }
  for (int64_t t = T_ - 1; t >= 0; --t) {
    const int64_t bm = (b * T_ + t) * M, bd = (b * T_ + t) * D;
    A kl[NL], ql[NL];
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t c = lane + 32 * j;
      kl[j] = c < M ? Elem<T>::ld(k + bm + c) : A(0);
      ql[j] = c < M ? Elem<T>::ld(q + bm + c) : A(0);
    }
#pragma unroll
    for (int o = 0; o < kOwn; ++o) {
      const int64_t row = r0 + o;
      const bool in = row < D;
      A s = A(0);
#pragma unroll
      for (int j = 0; j < NL; ++j) s += G[o][j] * kl[j];
      s = warp_sum(s);
      const A g = in ? Elem<T>::ld(go + bd + row) : A(0);
#pragma unroll
      for (int j = 0; j < NL; ++j) G[o][j] += g * ql[j] - s * kl[j];
      if (lane == 0 && in) {
        Elem<T>::st(dv + bd + row, s);
        dv_acc[bd + row] = s;
      }
    }
  }
#pragma unroll
  for (int o = 0; o < kOwn; ++o)
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t row = r0 + o, c = lane + 32 * j;
      if (row < D && c < M) Elem<T>::st(ds + (b * D + row) * M + c, G[o][j]);
    }
}

// columns: own = m, lanes over d.
template <typename T, int NL>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
dfw_bwd_cols_kernel(const T *__restrict__ go, const T *__restrict__ gs, const T *__restrict__ q,
                    const T *__restrict__ k, const typename Elem<T>::acc *__restrict__ delta,
                    const typename Elem<T>::acc *__restrict__ dv_acc, const T *__restrict__ fin,
                    T *__restrict__ dq, T *__restrict__ dk, int64_t B, int64_t T_, int64_t D,
                    int64_t M) {
  using A = typename Elem<T>::acc;
  const int lane = threadIdx.x & 31;
  const int64_t groups = (M + kOwn - 1) / kOwn;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (warp >= B * groups) return;
  const int64_t b = warp / groups;
  const int64_t m0 = (warp % groups) * kOwn;

  A G[kOwn][NL], S[kOwn][NL];
#pragma unroll
  for (int o = 0; o < kOwn; ++o)
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t m = m0 + o, d = lane + 32 * j;
      const bool in = m < M && d < D;
      G[o][j] = in ? Elem<T>::ld(gs + (b * D + d) * M + m) : A(0);
      S[o][j] = in ? Elem<T>::ld(fin + (b * D + d) * M + m) : A(0);
    }
  for (int64_t t = T_ - 1; t >= 0; --t) {
    const int64_t bm = (b * T_ + t) * M, bd = (b * T_ + t) * D;
    A dl[NL], dvv[NL], gl[NL];
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t d = lane + 32 * j;
      const bool in = d < D;
      dl[j] = in ? delta[bd + d] : A(0);
      dvv[j] = in ? dv_acc[bd + d] : A(0);
      gl[j] = in ? Elem<T>::ld(go + bd + d) : A(0);
    }
#pragma unroll
    for (int o = 0; o < kOwn; ++o) {
      const int64_t m = m0 + o;
      const bool in = m < M;
      const A km = in ? Elem<T>::ld(k + bm + m) : A(0);
      const A qm = in ? Elem<T>::ld(q + bm + m) : A(0);
      A aq = A(0), ak = A(0);
#pragma unroll
      for (int j = 0; j < NL; ++j) {
        const A sp = S[o][j] - dl[j] * km;  // S_{t-1}
        aq += gl[j] * sp;
        ak += dl[j] * G[o][j] - dvv[j] * sp;
        G[o][j] += gl[j] * qm - dvv[j] * km;
        S[o][j] = sp;
      }
      aq = warp_sum(aq);
      ak = warp_sum(ak);
      if (lane == 0 && in) {
        Elem<T>::st(dq + bm + m, aq);
        Elem<T>::st(dk + bm + m, ak);
      }
    }
  }
}

int pick_nl(int64_t extent) {
  const int64_t need = (extent + 31) / 32;
  for (int nl : {1, 2, 4, 8, 16})
    if (need <= nl) return nl;
  return 0;
}

template <typename T, int NL>
int fwd_nl(const void *q, const void *k, const void *v, const void *state, void *out, void *fin,
           void *delta, int64_t B, int64_t T_, int64_t D, int64_t M, cudaStream_t st) {
  using A = typename Elem<T>::acc;
  const int64_t grid = ceil_div64(B * ceil_div64(D, kOwn), kWarpsPerCta);
  dfw_fwd_kernel<T, NL><<<(unsigned)grid, kWarpsPerCta * 32, 0, st>>>(
      (const T *)q, (const T *)k, (const T *)v, (const T *)state, (T *)out, (T *)fin, (A *)delta,
      B, T_, D, M);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

template <typename T, int NLM, int NLD>
int bwd_nl(const void *go, const void *gs, const void *q, const void *k, const void *delta,
           const void *fin, void *dq, void *dk, void *dv, void *ds, void *dv_acc, int64_t B,
           int64_t T_, int64_t D, int64_t M, cudaStream_t st) {
  using A = typename Elem<T>::acc;
  const int64_t grid_r = ceil_div64(B * ceil_div64(D, kOwn), kWarpsPerCta);
  dfw_bwd_rows_kernel<T, NLM><<<(unsigned)grid_r, kWarpsPerCta * 32, 0, st>>>(
      (const T *)go, (const T *)gs, (const T *)q, (const T *)k, (T *)dv, (T *)ds, (A *)dv_acc, B,
      T_, D, M);
  T2FW_CHECK_LAUNCH(1);
  const int64_t grid_c = ceil_div64(B * ceil_div64(M, kOwn), kWarpsPerCta);
  dfw_bwd_cols_kernel<T, NLD><<<(unsigned)grid_c, kWarpsPerCta * 32, 0, st>>>(
      (const T *)go, (const T *)gs, (const T *)q, (const T *)k, (const A *)delta,
      (const A *)dv_acc, (const T *)fin, (T *)dq, (T *)dk, B, T_, D, M);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

template <typename T, int NLM>
int bwd_pick_d(int nld, const void *go, const void *gs, const void *q, const void *k,
               const void *delta, const void *fin, void *dq, void *dk, void *dv, void *ds,
               void *dv_acc, int64_t B, int64_t T_, int64_t D, int64_t M, cudaStream_t st) {
#define T2FW_CASE(N)                                                                             \
  case N:                                                                                        \
    return bwd_nl<T, NLM, N>(go, gs, q, k, delta, fin, dq, dk, dv, ds, dv_acc, B, T_, D, M, st);
  switch (nld) {
    T2FW_CASE(1) T2FW_CASE(2) T2FW_CASE(4) T2FW_CASE(8) T2FW_CASE(16)
  }
#undef T2FW_CASE
  return T2FW_ERR_UNSUPPORTED;
}

template <typename T>
int fwd_typed(const void *q, const void *k, const void *v, const void *state, void *out,
              void *fin, void *delta, int64_t B, int64_t T_, int64_t D, int64_t M,
              cudaStream_t st) {
  switch (pick_nl(M)) {
    case 1: return fwd_nl<T, 1>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
    case 2: return fwd_nl<T, 2>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
    case 4: return fwd_nl<T, 4>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
    case 8: return fwd_nl<T, 8>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
    case 16: return fwd_nl<T, 16>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
  }
  set_error("dfw forward: M=%lld exceeds the supported maximum of 512", (long long)M);
  return T2FW_ERR_UNSUPPORTED;
}

template <typename T>
int bwd_typed(const void *go, const void *gs, const void *q, const void *k, const void *delta,
              const void *fin, void *dq, void *dk, void *dv, void *ds, void *dv_acc, int64_t B,
              int64_t T_, int64_t D, int64_t M, cudaStream_t st) {
  const int nld = pick_nl(D);
  int rc = T2FW_ERR_UNSUPPORTED;
#define T2FW_CASE(N)                                                                             \
  case N:                                                                                        \
    rc = bwd_pick_d<T, N>(nld, go, gs, q, k, delta, fin, dq, dk, dv, ds, dv_acc, B, T_, D, M, st); \
    break;
  switch (pick_nl(M)) {
    T2FW_CASE(1) T2FW_CASE(2) T2FW_CASE(4) T2FW_CASE(8) T2FW_CASE(16)
  }
#undef T2FW_CASE
  if (rc == T2FW_ERR_UNSUPPORTED)
    set_error("dfw backward: D=%lld, M=%lld exceed the supported maximum of 512", (long long)D,
              (long long)M);
  return rc;
}

}  // namespace

int dfw_scan_forward(const void *q, const void *k, const void *v, const void *state, void *out,
                     void *fin, void *delta, int64_t B, int64_t T_, int64_t D, int64_t M,
                     int dtype, cudaStream_t st) {
  switch (dtype) {
    case T2FW_F16: return fwd_typed<__half>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
    case T2FW_BF16: return fwd_typed<__nv_bfloat16>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
    case T2FW_F32: return fwd_typed<float>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
    case T2FW_F64: return fwd_typed<double>(q, k, v, state, out, fin, delta, B, T_, D, M, st);
  }
  set_error("unknown dtype %d", dtype);
  return T2FW_ERR_BAD_ARG;
}

int dfw_scan_backward(const void *go, const void *gs, const void *q, const void *k,
                      const void *delta, const void *fin, void *dq, void *dk, void *dv, void *ds,
                      void *dv_acc, int64_t B, int64_t T_, int64_t D, int64_t M, int dtype,
                      cudaStream_t st) {
  switch (dtype) {
    case T2FW_F16:
      return bwd_typed<__half>(go, gs, q, k, delta, fin, dq, dk, dv, ds, dv_acc, B, T_, D, M, st);
    case T2FW_BF16:
      return bwd_typed<__nv_bfloat16>(go, gs, q, k, delta, fin, dq, dk, dv, ds, dv_acc, B, T_, D, M, st);
    case T2FW_F32:
      return bwd_typed<float>(go, gs, q, k, delta, fin, dq, dk, dv, ds, dv_acc, B, T_, D, M, st);
    case T2FW_F64:
      return bwd_typed<double>(go, gs, q, k, delta, fin, dq, dk, dv, ds, dv_acc, B, T_, D, M, st);
  }
  set_error("unknown dtype %d", dtype);
  return T2FW_ERR_BAD_ARG;
}

}  // namespace t2fw
