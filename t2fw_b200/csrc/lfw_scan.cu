// Decay-rule ("LFW") scan kernels: the shape- and dtype-general path.
//
//   S_t = (f_t fk_t^T) .* S_{t-1} + x_t k_t^T ,  o_t = S_t q_t
//
// One warp owns a few lines of the D x K state (rows in the "row" orientation, columns in the
// "column" orientation), the lanes spread along the other axis, and time is walked
// sequentially with the state in registers in the accumulation type (float, or double for
// double storage).  Every output of the reference's forward (scan kernel + einsum,
// t2fw/csrc/lfw_kernel.cu:18-59, t2fw/csrc/lfw.cpp:45) and backward (reverse scan + five
// einsums + two in-place multiplies, t2fw/csrc/lfw_kernel.cu:61-102, t2fw/csrc/lfw.cpp:84-93)
// is produced inside the kernels; no [B,T,D,K] tensor exists.  Only every C-th state is
// stored; the backward pass recomputes the others from those checkpoints.
//
// The backward runs the same kernel twice with the two axes exchanged:
//   row orientation    (own = d, lanes = k): d_x = R k, d_f = (R.*S_prev) fk, d_state
//   column orientation (own = k, lanes = d): d_k = R^T x, d_f_key = (R.*S_prev)^T f, d_q = S^T dO
// so every reduction is a warp reduction and the result is deterministic.
#include "common.cuh"

namespace t2fw {

namespace {

constexpr int kWarpsPerCta = 4;

template <typename T, int NL, int OWN>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
lfw_scan_fwd_kernel(const T *__restrict__ x, const T *__restrict__ f, const T *__restrict__ q,
                    const T *__restrict__ k, const T *__restrict__ fk,
                    const T *__restrict__ state, T *__restrict__ out, T *__restrict__ ckpt,
                    int64_t B, int64_t T_, int64_t D, int64_t K, int64_t C, int64_t nslots,
                    const int *__restrict__ rowflag) {
  using A = typename Elem<T>::acc;
  const int lane = threadIdx.x & 31;
  const int64_t groups = (D + OWN - 1) / OWN;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (warp >= B * groups) return;
  const int64_t b = warp / groups;
  const int64_t r0 = (warp % groups) * OWN;
  if (rowflag != nullptr && rowflag[b] == 0) return;  // only rows the caller marked

  A S[OWN][NL];
#pragma unroll
  for (int o = 0; o < OWN; ++o)
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t row = r0 + o, c = lane + 32 * j;
      S[o][j] = (row < D && c < K) ? Elem<T>::ld(state + (b * D + row) * K + c) : A(0);
    }

  for (int64_t t = 0; t < T_; ++t) {
    const int64_t bk = (b * T_ + t) * K, bd = (b * T_ + t) * D;
    A gl[NL], kl[NL], ql[NL];
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t c = lane + 32 * j;
      const bool in = c < K;
      gl[j] = in ? Elem<T>::ld(fk + bk + c) : A(0);
      kl[j] = in ? Elem<T>::ld(k + bk + c) : A(0);
      ql[j] = in ? Elem<T>::ld(q + bk + c) : A(0);
    }
#pragma unroll
    for (int o = 0; o < OWN; ++o) {
      const int64_t row = r0 + o;
      const bool in = row < D;
      const A xo = in ? Elem<T>::ld(x + bd + row) : A(0);
      const A ao = in ? Elem<T>::ld(f + bd + row) : A(0);
      A acc = A(0);
#pragma unroll
      for (int j = 0; j < NL; ++j) {
        S[o][j] = S[o][j] * (ao * gl[j]) + xo * kl[j];
        acc += S[o][j] * ql[j];
      }
      acc = warp_sum(acc);
      if (lane == 0 && in) Elem<T>::st(out + bd + row, acc);
    }
    if ((t + 1) % C == 0 || t == T_ - 1) {
      const int64_t slot = t / C;
#pragma unroll
      for (int o = 0; o < OWN; ++o)
#pragma unroll
        for (int j = 0; j < NL; ++j) {
          const int64_t row = r0 + o, c = lane + 32 * j;
          if (row < D && c < K)
            Elem<T>::st(ckpt + ((b * nslots + slot) * D + row) * K + c, S[o][j]);
        }
    }
  }
}

// Arguments of the orientation-agnostic backward kernel.  "own" is the axis whose lines a warp
// owns, "lane" the axis the lanes spread over.
template <typename T>
struct LineArgs {
  const T *xo, *go, *po;  // own-axis vectors  [B,T,NO]: (x, f, dO) or (k, fk, q)
  const T *xl, *gl, *pl;  // lane-axis vectors [B,T,NLn]: (k, fk, q) or (x, f, dO)
  T *d_xo;                // sum over lanes of R * xl             -> d_x  or d_k
  T *d_go;                // sum over lanes of R * S_prev * gl    -> d_f  or d_f_key
  T *d_po;                // sum over lanes of S_t * pl           -> d_q  (column orientation only)
  const T *state0, *ckpt, *grad_state;
  T *d_state;             // written by the row orientation only (may be null)
  int64_t B, T_, NO, NLn; // batch, time, own extent, lane extent
  int64_t so, sl;         // strides of the own / lane axis inside one [D,K] state
  int64_t C, nslots;      // checkpoint interval and slot count
  int seg;                // steps of state history kept in shared memory at once
  const int *rowflag;     // if not null, only batch rows with a non-zero flag are processed
};

template <typename T, int NL, int OWN, bool WITH_SP>
__global__ void __launch_bounds__(kWarpsPerCta * 32) lfw_line_bwd_kernel(const LineArgs<T> a) {
  using A = typename Elem<T>::acc;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31;
  const int wic = threadIdx.x >> 5;
  A *hist = reinterpret_cast<A *>(smem_raw) + (size_t)wic * a.seg * OWN * NL * 32;

  const int64_t groups = (a.NO + OWN - 1) / OWN;
  const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wic;
  if (warp >= a.B * groups) return;
  const int64_t b = warp / groups;
  const int64_t o0 = (warp % groups) * OWN;
  const int64_t DK = a.NO * a.NLn;
  if (a.rowflag != nullptr && a.rowflag[b] == 0) return;

  auto state_off = [&](int o, int j) { return (o0 + o) * a.so + (int64_t)(lane + 32 * j) * a.sl; };
  auto valid = [&](int o, int j) { return (o0 + o) < a.NO && (lane + 32 * j) < a.NLn; };

  A R[OWN][NL], S[OWN][NL];
#pragma unroll
  for (int o = 0; o < OWN; ++o)
#pragma unroll
    for (int j = 0; j < NL; ++j)
      R[o][j] = valid(o, j) ? Elem<T>::ld(a.grad_state + b * DK + state_off(o, j)) : A(0);

  // one forward step of the recurrence on the register tile
  auto fwd_step = [&](int64_t t) {
    const int64_t bo = (b * a.T_ + t) * a.NO, bl = (b * a.T_ + t) * a.NLn;
    A gl[NL], xl[NL];
#pragma unroll
    for (int j = 0; j < NL; ++j) {
      const int64_t c = lane + 32 * j;
      const bool in = c < a.NLn;
      gl[j] = in ? Elem<T>::ld(a.gl + bl + c) : A(0);
      xl[j] = in ? Elem<T>::ld(a.xl + bl + c) : A(0);
    }
#pragma unroll
    for (int o = 0; o < OWN; ++o) {
      const bool in = (o0 + o) < a.NO;
      const A xo = in ? Elem<T>::ld(a.xo + bo + o0 + o) : A(0);
      const A go = in ? Elem<T>::ld(a.go + bo + o0 + o) : A(0);
#pragma unroll
      for (int j = 0; j < NL; ++j) S[o][j] = S[o][j] * (go * gl[j]) + xo * xl[j];
    }
  };

  const int64_t nchunks = (a.T_ + a.C - 1) / a.C;
  for (int64_t c = nchunks - 1; c >= 0; --c) {
    const int64_t t0 = c * a.C;
    const int64_t t1 = (t0 + a.C < a.T_) ? t0 + a.C : a.T_;
    const int64_t nseg = (t1 - t0 + a.seg - 1) / a.seg;
    const T *src = (c == 0) ? a.state0 + b * DK : a.ckpt + (b * a.nslots + (c - 1)) * DK;
    for (int64_t sg = nseg - 1; sg >= 0; --sg) {
      const int64_t s0 = t0 + sg * a.seg;
      const int64_t s1 = (s0 + a.seg < t1) ? s0 + a.seg : t1;
#pragma unroll
      for (int o = 0; o < OWN; ++o)
#pragma unroll
        for (int j = 0; j < NL; ++j)
          S[o][j] = valid(o, j) ? Elem<T>::ld(src + state_off(o, j)) : A(0);
      for (int64_t t = t0; t < s0; ++t) fwd_step(t);
      for (int64_t t = s0; t < s1; ++t) {
#pragma unroll
        for (int o = 0; o < OWN; ++o)
#pragma unroll
          for (int j = 0; j < NL; ++j)
            hist[(((t - s0) * OWN + o) * NL + j) * 32 + lane] = S[o][j];
        fwd_step(t);
      }
      // S now holds the state after step s1-1; walk back to s0.
      for (int64_t t = s1 - 1; t >= s0; --t) {
        const int64_t bo = (b * a.T_ + t) * a.NO, bl = (b * a.T_ + t) * a.NLn;
        A gl[NL], xl[NL], pl[NL];
#pragma unroll
        for (int j = 0; j < NL; ++j) {
          const int64_t cc = lane + 32 * j;
          const bool in = cc < a.NLn;
          gl[j] = in ? Elem<T>::ld(a.gl + bl + cc) : A(0);
          xl[j] = in ? Elem<T>::ld(a.xl + bl + cc) : A(0);
          pl[j] = in ? Elem<T>::ld(a.pl + bl + cc) : A(0);
        }
#pragma unroll
        for (int o = 0; o < OWN; ++o) {
          const bool in = (o0 + o) < a.NO;
          const A go = in ? Elem<T>::ld(a.go + bo + o0 + o) : A(0);
          const A po = in ? Elem<T>::ld(a.po + bo + o0 + o) : A(0);
          A ax = A(0), ag = A(0), ap = A(0);
#pragma unroll
          for (int j = 0; j < NL; ++j) {
            const A sp = hist[(((t - s0) * OWN + o) * NL + j) * 32 + lane];
            const A r = R[o][j] + po * pl[j];   // gradient w.r.t. S_t
            ax += r * xl[j];
            ag += (r * sp) * gl[j];
            if (WITH_SP) ap += S[o][j] * pl[j];
            R[o][j] = r * (go * gl[j]);         // what flows on to S_{t-1}
            S[o][j] = sp;
          }
          ax = warp_sum(ax);
          ag = warp_sum(ag);
          if (WITH_SP) ap = warp_sum(ap);
          if (lane == 0 && in) {
            Elem<T>::st(a.d_xo + bo + o0 + o, ax);
            Elem<T>::st(a.d_go + bo + o0 + o, ag);
            if (WITH_SP) Elem<T>::st(a.d_po + bo + o0 + o, ap);
          }
        }
      }
    }
  }
  if (a.d_state != nullptr) {
#pragma unroll
    for (int o = 0; o < OWN; ++o)
#pragma unroll
      for (int j = 0; j < NL; ++j)
        if (valid(o, j)) Elem<T>::st(a.d_state + b * DK + state_off(o, j), R[o][j]);
  }
}

int pick_nl(int64_t extent) {
  const int64_t need = (extent + 31) / 32;
  for (int nl : {1, 2, 4, 8, 16})
    if (need <= nl) return nl;
  return 0;
}

template <typename T, int NL>
int launch_fwd(const void *x, const void *f, const void *q, const void *k, const void *fk,
               const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int64_t D,
               int64_t K, int64_t C, cudaStream_t st, const int *rowflag) {
  constexpr int OWN = 4;
  const int64_t warps = B * ceil_div64(D, OWN);
  const int64_t grid = ceil_div64(warps, kWarpsPerCta);
  lfw_scan_fwd_kernel<T, NL, OWN><<<(unsigned)grid, kWarpsPerCta * 32, 0, st>>>(
      (const T *)x, (const T *)f, (const T *)q, (const T *)k, (const T *)fk, (const T *)state,
      (T *)out, (T *)ckpt, B, T_, D, K, C, ceil_div64(T_, C), rowflag);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

template <typename T, int NL, bool WITH_SP>
int launch_line(LineArgs<T> a, cudaStream_t st) {
  constexpr int OWN = 2;
  using A = typename Elem<T>::acc;
  const size_t per_step = (size_t)kWarpsPerCta * OWN * NL * 32 * sizeof(A);
  int seg = (int)(49152 / per_step);
  if (seg > 16) seg = 16;
  if (seg < 1) seg = 1;
  a.seg = seg;
  const int64_t warps = a.B * ceil_div64(a.NO, OWN);
  const int64_t grid = ceil_div64(warps, kWarpsPerCta);
  lfw_line_bwd_kernel<T, NL, OWN, WITH_SP>
      <<<(unsigned)grid, kWarpsPerCta * 32, per_step * seg, st>>>(a);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

template <typename T>
int fwd_typed(const void *x, const void *f, const void *q, const void *k, const void *fk,
              const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int64_t D,
              int64_t K, int64_t C, cudaStream_t st, const int *rowflag) {
  switch (pick_nl(K)) {
    case 1: return launch_fwd<T, 1>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
    case 2: return launch_fwd<T, 2>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
    case 4: return launch_fwd<T, 4>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
    case 8: return launch_fwd<T, 8>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
    case 16: return launch_fwd<T, 16>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
  }
  set_error("lfw forward: K=%lld exceeds the supported maximum of 512", (long long)K);
  return T2FW_ERR_UNSUPPORTED;
}

template <typename T, bool WITH_SP>
int line_typed(const LineArgs<T> &a, cudaStream_t st) {
  switch (pick_nl(a.NLn)) {
    case 1: return launch_line<T, 1, WITH_SP>(a, st);
    case 2: return launch_line<T, 2, WITH_SP>(a, st);
    case 4: return launch_line<T, 4, WITH_SP>(a, st);
    case 8: return launch_line<T, 8, WITH_SP>(a, st);
    case 16: return launch_line<T, 16, WITH_SP>(a, st);
  }
  set_error("lfw backward: extent %lld exceeds the supported maximum of 512", (long long)a.NLn);
  return T2FW_ERR_UNSUPPORTED;
}

template <typename T>
int bwd_typed(const void *go, const void *gs, const void *x, const void *f, const void *q,
              const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
              void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B, int64_t T_, int64_t D,
              int64_t K, int64_t C, cudaStream_t st, const int *rowflag) {
  LineArgs<T> row{};
  row.xo = (const T *)x; row.go = (const T *)f; row.po = (const T *)go;
  row.xl = (const T *)k; row.gl = (const T *)fk; row.pl = (const T *)q;
  row.d_xo = (T *)dx; row.d_go = (T *)df; row.d_po = nullptr;
  row.state0 = (const T *)state; row.ckpt = (const T *)ckpt; row.grad_state = (const T *)gs;
  row.d_state = (T *)ds;
  row.B = B; row.T_ = T_; row.NO = D; row.NLn = K; row.so = K; row.sl = 1;
  row.C = C; row.nslots = ceil_div64(T_, C); row.rowflag = rowflag;
  int rc = line_typed<T, false>(row, st);
  if (rc != T2FW_OK) return rc;

  LineArgs<T> col{};
  col.xo = (const T *)k; col.go = (const T *)fk; col.po = (const T *)q;
  col.xl = (const T *)x; col.gl = (const T *)f; col.pl = (const T *)go;
  col.d_xo = (T *)dk; col.d_go = (T *)dfk; col.d_po = (T *)dq;
  col.state0 = (const T *)state; col.ckpt = (const T *)ckpt; col.grad_state = (const T *)gs;
  col.d_state = nullptr;
  col.B = B; col.T_ = T_; col.NO = K; col.NLn = D; col.so = 1; col.sl = K;
  col.C = C; col.nslots = ceil_div64(T_, C); col.rowflag = rowflag;
  return line_typed<T, true>(col, st);
}

}  // namespace

int lfw_scan_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                     const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int64_t D,
                     int64_t K, int dtype, int64_t C, cudaStream_t st, const int *rowflag) {
  switch (dtype) {
    case T2FW_F16: return fwd_typed<__half>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
    case T2FW_BF16: return fwd_typed<__nv_bfloat16>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
    case T2FW_F32: return fwd_typed<float>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
    case T2FW_F64: return fwd_typed<double>(x, f, q, k, fk, state, out, ckpt, B, T_, D, K, C, st, rowflag);
  }
  set_error("unknown dtype %d", dtype);
  return T2FW_ERR_BAD_ARG;
}

int lfw_scan_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                      const void *k, const void *fk, const void *state, const void *ckpt,
                      void *dx, void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B,
                      int64_t T_, int64_t D, int64_t K, int dtype, int64_t C, cudaStream_t st,
                      const int *rowflag) {
  if (D > 512 || K > 512) {
    set_error("lfw backward: D=%lld, K=%lld exceed the supported maximum of 512", (long long)D,
              (long long)K);
    return T2FW_ERR_UNSUPPORTED;
  }
  switch (dtype) {
    case T2FW_F16:
      return bwd_typed<__half>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds, B, T_, D, K, C, st, rowflag);
    case T2FW_BF16:
      return bwd_typed<__nv_bfloat16>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds, B, T_, D, K, C, st, rowflag);
    case T2FW_F32:
      return bwd_typed<float>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds, B, T_, D, K, C, st, rowflag);
    case T2FW_F64:
      return bwd_typed<double>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds, B, T_, D, K, C, st, rowflag);
  }
  set_error("unknown dtype %d", dtype);
  return T2FW_ERR_BAD_ARG;
}

}  // namespace t2fw
