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
#include "seq_layout.cuh"

namespace t2fw {

using namespace c64;

int lfw_chunk_local_umma(bool backward, const seq::Maps &mp, float *M, float *Ac, float *Gc, int *flags, int64_t BH,
                         int64_t T_, int dtype, cudaStream_t st);
int lfw_c64_forward_out(const seq::Maps &mp, const void *state, const void *ckpt, void *out, int64_t out_ld,
                        int out_col, int *rowflag, int64_t BH, int64_t T_, int dtype, cudaStream_t st);
int lfw_c64_backward_main(const seq::Maps &mp, const void *state, const void *ckpt, const float *Rend,
                          void *const outs[5], const int64_t out_ld[5], const int out_col[5], int *rowflag,
                          int64_t BH, int64_t T_, int dtype, cudaStream_t st);

namespace {

struct Scratch {
  float *M, *Ac, *Gc;
  int *flags, *rowflag;
  void *ck_all;      // 16-bit states after every chunk [B][nc][64][64]; only for checkpoint intervals > 64
};

inline size_t scratch_floats(int64_t B, int64_t nc) {
  return (size_t)B * nc * kDim * kDim + 2 * (size_t)B * nc * kDim + (size_t)B * nc + (size_t)B;
}

inline size_t scratch_bytes(int64_t B, int64_t nc, int64_t ckpt_every) {
  size_t n = align_up(scratch_floats(B, nc) * sizeof(float), 256);
  if (ckpt_every != kC) n += align_up((size_t)B * nc * kDim * kDim * 2, 256);
  return n;
}

inline Scratch carve(void *scratch, int64_t B, int64_t nc) {
  Scratch s;
  s.M = static_cast<float *>(scratch);
  s.Ac = s.M + (size_t)B * nc * kDim * kDim;
  s.Gc = s.Ac + (size_t)B * nc * kDim;
  s.flags = reinterpret_cast<int *>(s.Gc + (size_t)B * nc * kDim);
  s.rowflag = s.flags + (size_t)B * nc;
  s.ck_all = static_cast<unsigned char *>(scratch) + align_up(scratch_floats(B, nc) * sizeof(float), 256);
  return s;
}

constexpr int kBatch = 16;         // chunks whose loads are in flight together
constexpr int kCarryThreads = 256; // one block = 16 state rows (d) of one batch row, 4 columns (k) per thread
constexpr int kCarryRows = kCarryThreads / (kDim / 4);

template <typename T> struct Quad;
template <> struct Quad<__half> {
  static __device__ __forceinline__ float4 ld(const __half *p) {
    const uint2 u = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__half *p, float4 v) {
    uint2 u;
    *reinterpret_cast<__half2 *>(&u.x) = __floats2half2_rn(v.x, v.y);
    *reinterpret_cast<__half2 *>(&u.y) = __floats2half2_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = u;
  }
};
template <> struct Quad<__nv_bfloat16> {
  static __device__ __forceinline__ float4 ld(const __nv_bfloat16 *p) {
    const uint2 u = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void st(__nv_bfloat16 *p, float4 v) {
    uint2 u;
    *reinterpret_cast<__nv_bfloat162 *>(&u.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162 *>(&u.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = u;
  }
};

// One thread per (row, d, four consecutive k); a block covers 16 state rows of one batch row.  The
// recurrence over the chunks is a dependent chain, so the loads of up to 16 chunks are all issued
// before the chain starts (one round of memory latency per 16 chunks); the decay vectors of those
// chunks are shared by the block and go through shared memory.
//   kFwd:  S_{c+1} = (Ac Gc^T) S_c + L_c from the caller's state; checkpoint slot c = S_{c+1}
//   !kFwd: R_end(c-1) = (Ac Gc^T) R_end(c) + G_c from grad_state, last chunk first; G_c is
//          overwritten with R_end(c); the value left after chunk 0 is d_state
template <typename T, bool kFwd>
__global__ void __launch_bounds__(kCarryThreads, 3)
lfw_c64_carry_kernel(const T *__restrict__ init, float *__restrict__ M, const float *__restrict__ Ac,
                     const float *__restrict__ Gc, const int *__restrict__ flags, int *__restrict__ rowflag,
                     int keep_rowflag, T *__restrict__ out, int64_t B, int64_t nc) {
  __shared__ float a_s[kBatch][kCarryRows];
  __shared__ __align__(16) float g_s[kBatch][kDim];
  const int tid = threadIdx.x;
  dependency_wait();
  const int64_t b = blockIdx.x / (kDim / kCarryRows);
  const int d0 = (int)(blockIdx.x % (kDim / kCarryRows)) * kCarryRows;
  const int dl = tid / (kDim / 4), d = d0 + dl, k0 = (tid % (kDim / 4)) * 4;
  // init may be null: the carry then starts from zero (the summary of a sequence segment)
  float4 S = init != nullptr ? Quad<T>::ld(init + ((size_t)b * kDim + d) * kDim + k0) : make_float4(0.f, 0.f, 0.f, 0.f);
  int any = 0;
  for (int64_t c0 = 0; c0 < nc; c0 += kBatch) {
    float4 l[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      int64_t c = c0 + j < nc ? c0 + j : nc - 1;
      if (!kFwd) c = nc - 1 - c;
      l[j] = *reinterpret_cast<const float4 *>(M + (((size_t)b * nc + c) * kDim + d) * kDim + k0);
    }
    __syncthreads();      // the previous batch's decay vectors are no longer read
    for (int i = tid; i < kBatch * (kCarryRows + kDim); i += kCarryThreads) {
      const int j = i / (kCarryRows + kDim), r = i % (kCarryRows + kDim);
      int64_t c = c0 + j < nc ? c0 + j : nc - 1;
      if (!kFwd) c = nc - 1 - c;
      const size_t bc = (size_t)b * nc + c;
      if (r < kCarryRows) a_s[j][r] = Ac[bc * kDim + d0 + r];
      else g_s[j][r - kCarryRows] = Gc[bc * kDim + r - kCarryRows];
    }
    if (tid == 0 && d0 == 0)
      for (int j = 0; j < kBatch && c0 + j < nc; ++j) any |= flags[(size_t)b * nc + c0 + j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (c0 + j < nc) {
        const int64_t c = kFwd ? c0 + j : nc - 1 - (c0 + j);
        const size_t off = (((size_t)b * nc + c) * kDim + d) * kDim + k0;
        if (!kFwd) *reinterpret_cast<float4 *>(M + off) = S;
        const float a = a_s[j][dl];
        const float4 g = *reinterpret_cast<const float4 *>(&g_s[j][k0]);
        S.x = a * g.x * S.x + l[j].x;
        S.y = a * g.y * S.y + l[j].y;
        S.z = a * g.z * S.z + l[j].z;
        S.w = a * g.w * S.w + l[j].w;
        if (kFwd) Quad<T>::st(out + off, S);
      }
    }
  }
  if (!kFwd) Quad<T>::st(out + ((size_t)b * kDim + d) * kDim + k0, S);
  if (tid == 0 && d0 == 0) rowflag[b] = keep_rowflag ? (rowflag[b] | any) : any;
}

// Checkpoint interval of m chunks: slot j of the caller's checkpoints = state after chunk
// min((j + 1) m, nc) - 1 of the per-chunk states.
template <typename T>
__global__ void __launch_bounds__(256)
lfw_c64_pick_ckpt_kernel(const T *__restrict__ all, T *__restrict__ ckpt, int64_t B, int64_t nc, int64_t m,
                         int64_t slots) {
  constexpr int kVec = kDim * kDim / 8;      // 16-byte pieces of one state
  const int64_t n = B * slots * kVec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t v = i % kVec, j = (i / kVec) % slots, b = i / (kVec * slots);
    const int64_t c = ((j + 1) * m < nc ? (j + 1) * m : nc) - 1;
    reinterpret_cast<uint4 *>(ckpt)[(b * slots + j) * kVec + v] =
        reinterpret_cast<const uint4 *>(all)[(b * nc + c) * kVec + v];
  }
}

// One sequence tensor of a call: base pointer, width of a row (elements), column of sub-item 0,
// and which 64-column window sub-item h reads: (h / hdiv) % hmod (0, 0 = head h of `heads`).
struct Tensor2D {
  const void *p;
  int64_t width;
  int col;
  int hdiv = 0, hmod = 0;
};

// Tensor maps for a kernel whose inputs are `ts` (in the kernel's order); rows = batch items x T.
int build_maps(seq::Maps &mp, const Tensor2D *ts, int n, int64_t rows, int heads, int flags, float q_scale) {
  if (rows >= (1ll << 31) || rows * heads / kC + rows * heads >= (1ll << 31)) {
    set_error("chunked decay rule: batch x time = %lld rows exceed the copy engine's 31-bit coordinates", (long long)rows);
    return T2FW_ERR_UNSUPPORTED;
  }
  bool dense = heads == 1;
  for (int i = 0; i < n; ++i) dense = dense && (ts[i].p == nullptr || (ts[i].width == kDim && ts[i].col == 0));
  if (dense) flags |= seq::kContiguous;               // [rows][64] arrays: linear copies, no tensor maps needed
  for (int i = 0; i < n; ++i) {
    mp.col[i] = ts[i].col;
    mp.base[i] = ts[i].p;
    mp.hdiv[i] = ts[i].hdiv > 0 ? ts[i].hdiv : 1;
    mp.hmod[i] = ts[i].hmod > 0 ? ts[i].hmod : heads;
    if (ts[i].p == nullptr || dense) continue;        // constant tensor (unit forget gate) / no map needed
    bool shared = false;
    for (int j = 0; j < i && !shared; ++j)
      if (ts[j].p == ts[i].p && ts[j].width == ts[i].width) {
        mp.m[i] = mp.m[j];                            // several tensors inside one array
        shared = true;
      }
    if (!shared) {
      const int rc = seq::make_map(&mp.m[i], ts[i].p, (uint64_t)rows, (uint64_t)ts[i].width, (uint64_t)ts[i].width);
      if (rc != T2FW_OK) return rc;
    }
  }
  mp.heads = heads;
  mp.flags = flags;
  mp.q_scale = q_scale;
  return T2FW_OK;
}

// The tensors of a call, plain or fused: x, f, q, k, fk, dO in that order (f.p null = constant 1).
struct Call {
  Tensor2D x, f, q, k, fk, go;
  int64_t B, T_;        // batch items, steps;  problem rows BH = B * heads
  int heads, flags;
  float q_scale;
};

// The states after every chunk (16-bit) from the caller's state: local kernel + carry.
template <typename T>
int chunk_states(const Call &c, const Scratch &s, const void *state, T *ck_all, int dtype, cudaStream_t st) {
  const int64_t BH = c.B * c.heads, nc = ceil_div64(c.T_, kC), rows = c.B * c.T_;
  seq::Maps mp;
  const Tensor2D loc[4] = {c.x, c.f, c.k, c.fk};
  int rc = build_maps(mp, loc, 4, rows, c.heads, c.flags, 1.f);
  if (rc != T2FW_OK) return rc;
  rc = lfw_chunk_local_umma(false, mp, s.M, s.Ac, s.Gc, s.flags, BH, c.T_, dtype, st);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_CUDA(launch_dependent(lfw_c64_carry_kernel<T, true>, dim3((unsigned)(BH * (kDim / kCarryRows))),
                                   dim3(kCarryThreads), 0, st, (const T *)state, s.M, (const float *)s.Ac,
                                   (const float *)s.Gc, (const int *)s.flags, s.rowflag, 0, ck_all, BH, nc));
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

// ckpt_every = m * 64.  m = 1: the carry writes the caller's checkpoints directly.  m > 1: the
// per-chunk states go to scratch and every m-th one (and the last) is copied out.
template <typename T>
int forward_typed(const Call &c, const void *state, void *out, int64_t out_ld, int out_col, void *ckpt, int dtype,
                  int64_t ckpt_every, void *scratch, cudaStream_t st) {
  const int64_t BH = c.B * c.heads, nc = ceil_div64(c.T_, kC), rows = c.B * c.T_, m = ckpt_every / kC;
  Scratch s = carve(scratch, BH, nc);
  T *ck_all = m == 1 ? (T *)ckpt : (T *)s.ck_all;
  int rc = chunk_states<T>(c, s, state, ck_all, dtype, st);
  if (rc != T2FW_OK) return rc;
  seq::Maps mp;
  const Tensor2D all[5] = {c.x, c.f, c.q, c.k, c.fk};
  rc = build_maps(mp, all, 5, rows, c.heads, c.flags, c.q_scale);
  if (rc != T2FW_OK) return rc;
  rc = lfw_c64_forward_out(mp, state, ck_all, out, out_ld, out_col, s.rowflag, BH, c.T_, dtype, st);
  if (rc != T2FW_OK || m == 1) return rc;
  const int64_t slots = ceil_div64(c.T_, ckpt_every), n = BH * slots * (kDim * kDim / 8);
  const int64_t blocks = ceil_div64(n, 256);
  lfw_c64_pick_ckpt_kernel<T><<<(unsigned)(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, st>>>(
      ck_all, (T *)ckpt, BH, nc, m, slots);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

// ckpt_every > 64: the states at the chunk starts that the caller's checkpoints do not hold are
// rebuilt from the caller's state first, exactly as the forward call built them.
template <typename T>
int backward_typed(const Call &c, const void *gs, const void *state, const void *ckpt, void *const outs[5],
                   const int64_t out_ld[5], const int out_col[5], void *ds, int dtype, int64_t ckpt_every,
                   void *scratch, cudaStream_t st) {
  const int64_t BH = c.B * c.heads, nc = ceil_div64(c.T_, kC), rows = c.B * c.T_, m = ckpt_every / kC;
  Scratch s = carve(scratch, BH, nc);
  if (m > 1) {
    const int rc0 = chunk_states<T>(c, s, state, (T *)s.ck_all, dtype, st);
    if (rc0 != T2FW_OK) return rc0;
    ckpt = s.ck_all;
  }
  seq::Maps mp;
  const Tensor2D loc[4] = {c.go, c.f, c.q, c.fk};
  int rc = build_maps(mp, loc, 4, rows, c.heads, c.flags, c.q_scale);
  if (rc != T2FW_OK) return rc;
  rc = lfw_chunk_local_umma(true, mp, s.M, s.Ac, s.Gc, s.flags, BH, c.T_, dtype, st);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_CUDA(launch_dependent(lfw_c64_carry_kernel<T, false>, dim3((unsigned)(BH * (kDim / kCarryRows))),
                                   dim3(kCarryThreads), 0, st, (const T *)gs, s.M, (const float *)s.Ac,
                                   (const float *)s.Gc, (const int *)s.flags, s.rowflag, m > 1 ? 1 : 0, (T *)ds, BH,
                                   nc));
  T2FW_CHECK_LAUNCH(1);
  const Tensor2D all[6] = {c.x, c.f, c.q, c.k, c.fk, c.go};
  rc = build_maps(mp, all, 6, rows, c.heads, c.flags, c.q_scale);
  if (rc != T2FW_OK) return rc;
  return lfw_c64_backward_main(mp, state, ckpt, s.M, outs, out_ld, out_col, s.rowflag, BH, c.T_, dtype, st);
}

Call plain_call(const void *x, const void *f, const void *q, const void *k, const void *fk, const void *go, int64_t B,
                int64_t T_) {
  Call c;
  c.x = {x, kDim, 0}; c.f = {f, kDim, 0}; c.q = {q, kDim, 0}; c.k = {k, kDim, 0}; c.fk = {fk, kDim, 0};
  c.go = {go, kDim, 0};
  c.B = B; c.T_ = T_; c.heads = 1; c.flags = 0; c.q_scale = 1.f;
  return c;
}

// A D x K state cut into (D/64) x (K/64) blocks: sub-item h = i * nk + j of a batch item is block
// (i, j); the d-side tensors [B*T][D] are read at window i, the k-side tensors [B*T][K] at window j,
// and every sub-item writes its own [T][64] result arrays (summed over the other index afterwards).
Call grid_call(const void *x, const void *f, const void *q, const void *k, const void *fk, const void *go, int64_t B,
               int64_t T_, int nd, int nk) {
  const int64_t D = (int64_t)nd * kDim, K = (int64_t)nk * kDim;
  Call c;
  c.x = {x, D, 0, nk, nd}; c.f = {f, D, 0, nk, nd}; c.go = {go, D, 0, nk, nd};
  c.q = {q, K, 0, 1, nk}; c.k = {k, K, 0, 1, nk}; c.fk = {fk, K, 0, 1, nk};
  c.B = B; c.T_ = T_; c.heads = nd * nk; c.flags = seq::kOutByRow; c.q_scale = 1.f;
  return c;
}

// fused layer: qkvg [B][T][4 * H * 64] = query | key | value | gate pre-activation, heads inside a row
Call fused_call(const void *qkvg, const void *go, int64_t B, int64_t T_, int H) {
  const int64_t C = (int64_t)H * kDim;
  Call c;
  c.q = {qkvg, 4 * C, 0}; c.k = {qkvg, 4 * C, (int)C}; c.x = {qkvg, 4 * C, (int)(2 * C)};
  c.fk = {qkvg, 4 * C, (int)(3 * C)};
  c.f = {nullptr, 0, 0};
  c.go = {go, C, 0};
  c.B = B; c.T_ = T_; c.heads = H; c.flags = seq::kUnitForget | seq::kSigmoidGate; c.q_scale = 0.125f;   // 1 / sqrt(64)
  return c;
}

}  // namespace

bool lfw_chunk_supported(int64_t D, int64_t K, int dtype, int64_t ckpt_every) {
  return D == kDim && K == kDim && ckpt_every >= kC && ckpt_every % kC == 0 &&
         (dtype == T2FW_F16 || dtype == T2FW_BF16);
}

size_t lfw_chunk_forward_scratch_bytes(int64_t B, int64_t T_, int64_t ckpt_every) {
  return scratch_bytes(B, ceil_div64(T_, kC), ckpt_every);
}

size_t lfw_chunk_backward_scratch_bytes(int64_t B, int64_t T_, int64_t ckpt_every) {
  return scratch_bytes(B, ceil_div64(T_, kC), ckpt_every);
}

// Both calls need every pointer 16-byte aligned (the C ABI routes other callers to the scan
// kernels).
int lfw_chunk_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                      const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int dtype,
                      int64_t ckpt_every, void *scratch, cudaStream_t st, const int **rowflag_out) {
  if (rowflag_out) *rowflag_out = carve(scratch, B, ceil_div64(T_, kC)).rowflag;
  const Call c = plain_call(x, f, q, k, fk, nullptr, B, T_);
  if (dtype == T2FW_F16) return forward_typed<__half>(c, state, out, kDim, 0, ckpt, dtype, ckpt_every, scratch, st);
  return forward_typed<__nv_bfloat16>(c, state, out, kDim, 0, ckpt, dtype, ckpt_every, scratch, st);
}

int lfw_chunk_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                       const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
                       void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B, int64_t T_,
                       int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st, const int **rowflag_out) {
  if (rowflag_out) *rowflag_out = carve(scratch, B, ceil_div64(T_, kC)).rowflag;
  const Call c = plain_call(x, f, q, k, fk, go, B, T_);
  void *const outs[5] = {dx, df, dq, dk, dfk};
  const int64_t ld[5] = {kDim, kDim, kDim, kDim, kDim};
  const int col[5] = {0, 0, 0, 0, 0};
  if (dtype == T2FW_F16)
    return backward_typed<__half>(c, gs, state, ckpt, outs, ld, col, ds, dtype, ckpt_every, scratch, st);
  return backward_typed<__nv_bfloat16>(c, gs, state, ckpt, outs, ld, col, ds, dtype, ckpt_every, scratch, st);
}

// ---- block-grid form: inputs dense [B*T][D] / [B*T][K], states, checkpoints and results per block ----
int lfw_chunk_forward_grid(const void *x, const void *f, const void *q, const void *k, const void *fk,
                           const void *state_blocks, void *out_blocks, void *ckpt_blocks, int64_t B, int64_t T_,
                           int nd, int nk, int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st,
                           const int **rowflag_out) {
  const int64_t VB = B * nd * nk;
  if (rowflag_out) *rowflag_out = carve(scratch, VB, ceil_div64(T_, kC)).rowflag;
  const Call c = grid_call(x, f, q, k, fk, nullptr, B, T_, nd, nk);
  if (dtype == T2FW_F16)
    return forward_typed<__half>(c, state_blocks, out_blocks, kDim, 0, ckpt_blocks, dtype, ckpt_every, scratch, st);
  return forward_typed<__nv_bfloat16>(c, state_blocks, out_blocks, kDim, 0, ckpt_blocks, dtype, ckpt_every, scratch, st);
}

int lfw_chunk_backward_grid(const void *go, const void *gs_blocks, const void *x, const void *f, const void *q,
                            const void *k, const void *fk, const void *state_blocks, const void *ckpt_blocks,
                            void *dx, void *df, void *dq, void *dk, void *dfk, void *ds_blocks, int64_t B, int64_t T_,
                            int nd, int nk, int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st,
                            const int **rowflag_out) {
  const int64_t VB = B * nd * nk;
  if (rowflag_out) *rowflag_out = carve(scratch, VB, ceil_div64(T_, kC)).rowflag;
  const Call c = grid_call(x, f, q, k, fk, go, B, T_, nd, nk);
  void *const outs[5] = {dx, df, dq, dk, dfk};
  const int64_t ld[5] = {kDim, kDim, kDim, kDim, kDim};
  const int col[5] = {0, 0, 0, 0, 0};
  if (dtype == T2FW_F16)
    return backward_typed<__half>(c, gs_blocks, state_blocks, ckpt_blocks, outs, ld, col, ds_blocks, dtype, ckpt_every,
                                  scratch, st);
  return backward_typed<__nv_bfloat16>(c, gs_blocks, state_blocks, ckpt_blocks, outs, ld, col, ds_blocks, dtype,
                                       ckpt_every, scratch, st);
}

// ---- summary of a sequence segment (for splitting the time axis over devices) ------------------
// Total decay of a segment per feature: the product of the chunks' decay vectors.  A row with a
// flagged chunk (gate products beyond 2^100) gets NaN decays, so that whatever is built on the
// summary shows the problem instead of hiding it.
__global__ void __launch_bounds__(128)
lfw_c64_decay_totals_kernel(const float *__restrict__ Ac, const float *__restrict__ Gc, const int *__restrict__ rowflag,
                            float *__restrict__ A_out, float *__restrict__ G_out, int64_t B, int64_t nc) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * 2 * kDim) return;
  const int64_t b = i / (2 * kDim);
  const int side = (int)((i / kDim) & 1), feat = (int)(i % kDim);
  const float *src = side ? Gc : Ac;
  float p = 1.f;
  for (int64_t c = 0; c < nc; ++c) p *= src[((size_t)b * nc + c) * kDim + feat];
  if (rowflag[b] != 0) p = __int_as_float(0x7fc00000);
  (side ? G_out : A_out)[b * kDim + feat] = p;
}

template <typename T>
int summary_typed(bool backward, const void *val_d, const void *gate_d, const void *val_k, const void *gate_k,
                  void *end_state, float *A_out, float *G_out, int64_t B, int64_t T_, int dtype, void *scratch,
                  cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC), rows = B * T_;
  Scratch s = carve(scratch, B, nc);
  seq::Maps mp;
  const Tensor2D loc[4] = {{val_d, kDim, 0}, {gate_d, kDim, 0}, {val_k, kDim, 0}, {gate_k, kDim, 0}};
  int rc = build_maps(mp, loc, 4, rows, 1, 0, 1.f);
  if (rc != T2FW_OK) return rc;
  rc = lfw_chunk_local_umma(backward, mp, s.M, s.Ac, s.Gc, s.flags, B, T_, dtype, st);
  if (rc != T2FW_OK) return rc;
  const dim3 grid((unsigned)(B * (kDim / kCarryRows)));
  if (backward) {      // the state gradient at the segment start that the segment's own output gradients cause
    T2FW_CHECK_CUDA(launch_dependent(lfw_c64_carry_kernel<T, false>, grid, dim3(kCarryThreads), 0, st, (const T *)nullptr,
                                     s.M, (const float *)s.Ac, (const float *)s.Gc, (const int *)s.flags, s.rowflag, 0,
                                     (T *)end_state, B, nc));
  } else {             // the state at the segment end that the segment's own inputs cause
    T2FW_CHECK_CUDA(launch_dependent(lfw_c64_carry_kernel<T, true>, grid, dim3(kCarryThreads), 0, st, (const T *)nullptr,
                                     s.M, (const float *)s.Ac, (const float *)s.Gc, (const int *)s.flags, s.rowflag, 0,
                                     (T *)s.ck_all, B, nc));
    lfw_c64_pick_ckpt_kernel<T><<<(unsigned)ceil_div64(B * (kDim * kDim / 8), 256), 256, 0, st>>>(
        (const T *)s.ck_all, (T *)end_state, B, nc, nc, 1);
  }
  lfw_c64_decay_totals_kernel<<<(unsigned)ceil_div64(B * 2 * kDim, 128), 128, 0, st>>>(s.Ac, s.Gc, s.rowflag, A_out,
                                                                                     G_out, B, nc);
  T2FW_CHECK_LAUNCH(backward ? 2 : 3);
  return T2FW_OK;
}

size_t lfw_segment_summary_scratch_bytes(int64_t B, int64_t T_) { return scratch_bytes(B, ceil_div64(T_, kC), 2 * kC); }

// forward flavour: (val_d, gate_d, val_k, gate_k) = (x, f, k, f_key), end_state = the state a zero state becomes over
// the segment; backward flavour: (dO, f, q, f_key), end_state = the state gradient at the segment start for a zero
// gradient at its end.  A_out, G_out [B][64] fp32: the segment's total decays.
int lfw_segment_summary(bool backward, const void *val_d, const void *gate_d, const void *val_k, const void *gate_k,
                        void *end_state, float *A_out, float *G_out, int64_t B, int64_t T_, int dtype, void *scratch,
                        cudaStream_t st) {
  if (dtype == T2FW_F16)
    return summary_typed<__half>(backward, val_d, gate_d, val_k, gate_k, end_state, A_out, G_out, B, T_, dtype, scratch, st);
  return summary_typed<__nv_bfloat16>(backward, val_d, gate_d, val_k, gate_k, end_state, A_out, G_out, B, T_, dtype,
                                      scratch, st);
}

// ---- fused layer entry points (heads read in place from the projection output) ----------------
size_t lfw_fused_scratch_bytes(int64_t B, int64_t T_, int H) { return lfw_chunk_forward_scratch_bytes(B * H, T_, kC); }

int lfw_fused_forward(const void *qkvg, const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int H,
                      int dtype, void *scratch, cudaStream_t st) {
  const Call c = fused_call(qkvg, nullptr, B, T_, H);
  const int64_t C = (int64_t)H * kDim;
  if (dtype == T2FW_F16) return forward_typed<__half>(c, state, out, C, 0, ckpt, dtype, kC, scratch, st);
  return forward_typed<__nv_bfloat16>(c, state, out, C, 0, ckpt, dtype, kC, scratch, st);
}

int lfw_fused_backward(const void *go, const void *gs, const void *qkvg, const void *state, const void *ckpt,
                       void *d_qkvg, void *ds, int64_t B, int64_t T_, int H, int dtype, void *scratch,
                       cudaStream_t st) {
  const Call c = fused_call(qkvg, go, B, T_, H);
  const int64_t C = (int64_t)H * kDim;
  // gradients land in d_qkvg [B][T][4C]: query | key | value | gate; there is no forget tensor
  void *const outs[5] = {d_qkvg, nullptr, d_qkvg, d_qkvg, d_qkvg};
  const int64_t ld[5] = {4 * C, 0, 4 * C, 4 * C, 4 * C};
  const int col[5] = {(int)(2 * C), 0, 0, (int)C, (int)(3 * C)};
  if (dtype == T2FW_F16) return backward_typed<__half>(c, gs, state, ckpt, outs, ld, col, ds, dtype, kC, scratch, st);
  return backward_typed<__nv_bfloat16>(c, gs, state, ckpt, outs, ld, col, ds, dtype, kC, scratch, st);
}

}  // namespace t2fw
