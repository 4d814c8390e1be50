// Chunked decay rule for D = K = 64, 16-bit storage, checkpoint interval 64: the carry over the
// chunks and the launch sequences of the forward and the backward call.
//
// Forward (replaces t2fw/csrc/lfw_kernel.cu:18-59 and the output einsum t2fw/csrc/lfw.cpp:45):
//   1. lfw_c64_local_kernel<.., true>   per (row, chunk): L_c, the chunk's own contribution to the
//      state at its end, and the chunk's total decay vectors
//   2. lfw_c64_carry_fwd_kernel         elementwise over chunks: S_{c+1} = (Ac Gc^T) .* S_c + L_c, written
//      as the 16-bit checkpoints (slot c = state after chunk c; the last slot is the next state)
//   3. lfw_c64_fwd_kernel               per (row, chunk): the outputs from the chunk's start state
// Backward (replaces t2fw/csrc/lfw_kernel.cu:61-102 and t2fw/csrc/lfw.cpp:84-93):
//   1. lfw_c64_local_kernel<.., false>  G_c, the chunk's own contribution to the state gradient at its start
//   2. lfw_c64_carry_bwd_kernel         from the last chunk down: R_end(c-1) = (Ac Gc^T) .* R_end(c) + G_c,
//      stored in place of G_c (fp32); what is left after chunk 0 is d_state
//   3. lfw_c64_bwd_kernel               per (row, chunk): d_x, d_f, d_q, d_k, d_f_key
// Scratch (floats): M[B][nc][64][64] | Ac[B][nc][64] | Gc[B][nc][64] | flags[B][nc] (int) |
// rowflag[B] (int).  A flagged batch row (gate products outside the range of the factored form) is
// recomputed by the scan kernels afterwards.
#include "lfw_c64.cuh"

namespace t2fw {

using namespace c64;

int lfw_c64_forward_out(const void *x, const void *f, const void *q, const void *k, const void *fk,
                        const void *state, const void *ckpt, void *out, int *rowflag, int64_t B, int64_t T_,
                        int dtype, cudaStream_t st);
int lfw_c64_backward_main(const void *go, const void *x, const void *f, const void *q, const void *k,
                          const void *fk, const void *state, const void *ckpt, const float *Rend, void *dx,
                          void *df, void *dq, void *dk, void *dfk, int *rowflag, int64_t B, int64_t T_,
                          int dtype, cudaStream_t st);

namespace {

struct Scratch {
  float *M, *Ac, *Gc;
  int *flags, *rowflag;
};

inline size_t scratch_floats(int64_t B, int64_t nc) {
  return (size_t)B * nc * kDim * kDim + 2 * (size_t)B * nc * kDim + (size_t)B * nc + (size_t)B;
}

inline Scratch carve(void *scratch, int64_t B, int64_t nc) {
  Scratch s;
  s.M = static_cast<float *>(scratch);
  s.Ac = s.M + (size_t)B * nc * kDim * kDim;
  s.Gc = s.Ac + (size_t)B * nc * kDim;
  s.flags = reinterpret_cast<int *>(s.Gc + (size_t)B * nc * kDim);
  s.rowflag = s.flags + (size_t)B * nc;
  return s;
}

template <typename T> struct Pair2;
template <> struct Pair2<__half> {
  static __device__ __forceinline__ float2 ld(const __half *p) { return __half22float2(*reinterpret_cast<const __half2 *>(p)); }
  static __device__ __forceinline__ void st(__half *p, float a, float b) { *reinterpret_cast<__half2 *>(p) = __floats2half2_rn(a, b); }
};
template <> struct Pair2<__nv_bfloat16> {
  static __device__ __forceinline__ float2 ld(const __nv_bfloat16 *p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p)); }
  static __device__ __forceinline__ void st(__nv_bfloat16 *p, float a, float b) { *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(a, b); }
};

constexpr int kBatch = 16;     // chunks whose loads are in flight together

// One thread per (row, d, two consecutive k).  The recurrence over the chunks is a dependent chain,
// so the loads of up to 16 chunks are all issued before the chain starts: one round of memory
// latency per 16 chunks.
//   kFwd:  S_{c+1} = (Ac Gc^T) S_c + L_c from the caller's state; checkpoint slot c = S_{c+1}
//   !kFwd: R_end(c-1) = (Ac Gc^T) R_end(c) + G_c from grad_state, last chunk first; G_c is
//          overwritten with R_end(c); the value left after chunk 0 is d_state
template <typename T, bool kFwd>
__global__ void __launch_bounds__(256)
lfw_c64_carry_kernel(const T *__restrict__ init, float *__restrict__ M, const float *__restrict__ Ac,
                     const float *__restrict__ Gc, const int *__restrict__ flags, int *__restrict__ rowflag,
                     T *__restrict__ out, int64_t B, int64_t nc) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * kDim * (kDim / 2)) return;
  const int64_t b = idx / (kDim * (kDim / 2));
  const int d = (int)((idx / (kDim / 2)) % kDim);
  const int k0 = (int)(idx % (kDim / 2)) * 2;
  const float2 s0 = Pair2<T>::ld(init + ((size_t)b * kDim + d) * kDim + k0);
  float S0 = s0.x, S1 = s0.y;
  int any = 0;
  for (int64_t c0 = 0; c0 < nc; c0 += kBatch) {
    float2 l[kBatch], gg[kBatch];
    float a[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      int64_t c = c0 + j < nc ? c0 + j : nc - 1;
      if (!kFwd) c = nc - 1 - c;
      const size_t bc = (size_t)b * nc + c;
      l[j] = *reinterpret_cast<const float2 *>(M + (bc * kDim + d) * kDim + k0);
      a[j] = Ac[bc * kDim + d];
      gg[j] = *reinterpret_cast<const float2 *>(Gc + bc * kDim + k0);
      if (d == 0 && k0 == 0) any |= flags[bc];
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (c0 + j < nc) {
        const int64_t c = kFwd ? c0 + j : nc - 1 - (c0 + j);
        const size_t bc = (size_t)b * nc + c;
        if (!kFwd) *reinterpret_cast<float2 *>(M + (bc * kDim + d) * kDim + k0) = make_float2(S0, S1);
        S0 = a[j] * gg[j].x * S0 + l[j].x;
        S1 = a[j] * gg[j].y * S1 + l[j].y;
        if (kFwd) Pair2<T>::st(out + (bc * kDim + d) * kDim + k0, S0, S1);
      }
    }
  }
  if (!kFwd) Pair2<T>::st(out + ((size_t)b * kDim + d) * kDim + k0, S0, S1);
  if (d == 0 && k0 == 0) rowflag[b] = any;
}

template <typename T>
int forward_typed(const void *x, const void *f, const void *q, const void *k, const void *fk, const void *state,
                  void *out, void *ckpt, int64_t B, int64_t T_, int dtype, void *scratch, cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC);
  Scratch s = carve(scratch, B, nc);
  int rc = lfw_chunk_local_umma(false, x, f, k, fk, s.M, s.Ac, s.Gc, s.flags, B, T_, dtype, st);
  if (rc != T2FW_OK) return rc;
  const int64_t n_carry = B * kDim * (kDim / 2);
  lfw_c64_carry_kernel<T, true><<<(unsigned)ceil_div64(n_carry, 256), 256, 0, st>>>(
      (const T *)state, s.M, s.Ac, s.Gc, s.flags, s.rowflag, (T *)ckpt, B, nc);
  T2FW_CHECK_LAUNCH(1);
  return lfw_c64_forward_out(x, f, q, k, fk, state, ckpt, out, s.rowflag, B, T_, dtype, st);
}

template <typename T>
int backward_typed(const void *go, const void *gs, const void *x, const void *f, const void *q, const void *k,
                   const void *fk, const void *state, const void *ckpt, void *dx, void *df, void *dq, void *dk,
                   void *dfk, void *ds, int64_t B, int64_t T_, int dtype, void *scratch, cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC);
  Scratch s = carve(scratch, B, nc);
  int rc = lfw_chunk_local_umma(true, go, f, q, fk, s.M, s.Ac, s.Gc, s.flags, B, T_, dtype, st);
  if (rc != T2FW_OK) return rc;
  const int64_t n_carry = B * kDim * (kDim / 2);
  lfw_c64_carry_kernel<T, false><<<(unsigned)ceil_div64(n_carry, 256), 256, 0, st>>>(
      (const T *)gs, s.M, s.Ac, s.Gc, s.flags, s.rowflag, (T *)ds, B, nc);
  T2FW_CHECK_LAUNCH(1);
  return lfw_c64_backward_main(go, x, f, q, k, fk, state, ckpt, s.M, dx, df, dq, dk, dfk, s.rowflag, B, T_, dtype, st);
}

}  // namespace

bool lfw_chunk_supported(int64_t D, int64_t K, int dtype, int64_t ckpt_every) {
  return D == kDim && K == kDim && ckpt_every == kC && (dtype == T2FW_F16 || dtype == T2FW_BF16);
}

size_t lfw_chunk_forward_scratch_bytes(int64_t B, int64_t T_) {
  return align_up(scratch_floats(B, ceil_div64(T_, kC)) * sizeof(float), 256);
}

size_t lfw_chunk_backward_scratch_bytes(int64_t B, int64_t T_) {
  return align_up(scratch_floats(B, ceil_div64(T_, kC)) * sizeof(float), 256);
}

// Both calls need every pointer 16-byte aligned (the C ABI routes other callers to the scan
// kernels) and return T2FW_ERR_UNSUPPORTED otherwise.
int lfw_chunk_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                      const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int dtype,
                      void *scratch, cudaStream_t st, const int **rowflag_out) {
  if (rowflag_out) *rowflag_out = carve(scratch, B, ceil_div64(T_, kC)).rowflag;
  if (dtype == T2FW_F16) return forward_typed<__half>(x, f, q, k, fk, state, out, ckpt, B, T_, dtype, scratch, st);
  return forward_typed<__nv_bfloat16>(x, f, q, k, fk, state, out, ckpt, B, T_, dtype, scratch, st);
}

int lfw_chunk_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                       const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
                       void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B, int64_t T_,
                       int dtype, void *scratch, cudaStream_t st, const int **rowflag_out) {
  if (rowflag_out) *rowflag_out = carve(scratch, B, ceil_div64(T_, kC)).rowflag;
  if (dtype == T2FW_F16)
    return backward_typed<__half>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds, B, T_, dtype, scratch, st);
  return backward_typed<__nv_bfloat16>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds, B, T_, dtype,
                                       scratch, st);
}

}  // namespace t2fw
