// Decay rule for state shapes larger than 64 x 64 (D, K multiples of 64, 16-bit storage).
//
// The recurrence S[d,k] <- f[d] fk[k] S[d,k] + x[d] k[k] never mixes state rows or columns, so
// a D x K state is a (D/64) x (K/64) grid of independent 64 x 64 blocks: block (i, j) sees the
// d-side vectors (x, f, dO) restricted to slice i and the k-side vectors (q, k, fk) restricted
// to slice j.  Everything that leaves the state is a sum over the other axis' blocks:
//   outputs, d_x, d_f  [.., slice i] = sum over j of block (i, j)'s result
//   d_q, d_k, d_f_key  [.., slice j] = sum over i of block (i, j)'s result
// while checkpoints, next state and d_state are block-local.  The blocks form a virtual batch of
// B * (D/64) * (K/64) problem rows for the chunked 64 x 64 kernels, which read each block's
// 64-column window of the caller's [B*T][D] / [B*T][K] arrays in place (tensor-map copies) and write
// per-block result arrays; those are summed in fp32 over the other axis' blocks.  Only the states and
// checkpoints are re-laid out per block.  For blocks the chunk kernels flag, contiguous copies of
// the windows are gathered and the scan kernels redo them.  This is what makes the long-sequence
// configuration (D = K = 128, T = 16384) run on the tensor-core path.
#include <type_traits>

#include "lfw_chunk.cuh"

namespace t2fw {

using namespace chunk;

namespace {

constexpr int kBlk = 64;

// dst[((b*nd + i)*nk + j)][t][0..63] = src[b][t][sel*64 ..], sel = i (d side) or j (k side), for the
// blocks whose flag is set (the ones the scan kernels have to redo; the chunk kernels read the
// windows in place).  A CTA takes (block, slice of the steps) items, so that in the usual case
// (no flag set) every CTA leaves after a few flag reads.
constexpr int kGatherSlices = 16;
template <typename T>
__global__ void __launch_bounds__(256)
gather_vec_kernel(const T *__restrict__ src, T *__restrict__ dst, int64_t B, int64_t T_, int W, int nd,
                  int nk, int dside, const int *__restrict__ rowflag) {
  const int64_t VB = B * nd * nk, per = (T_ + kGatherSlices - 1) / kGatherSlices;
  for (int64_t item = blockIdx.x; item < VB * kGatherSlices; item += gridDim.x) {
    const int64_t vb = item / kGatherSlices, t0 = (item % kGatherSlices) * per;
    if (rowflag[vb] == 0) continue;
    const int j = (int)(vb % nk), i = (int)((vb / nk) % nd);
    const int64_t b = vb / ((int64_t)nk * nd), t1 = t0 + per < T_ ? t0 + per : T_;
    const int sel = dside ? i : j;
    for (int64_t e = threadIdx.x; e < (t1 - t0) * (kBlk / 8); e += blockDim.x) {
      const int64_t t = t0 + e / (kBlk / 8);
      const int ch = (int)(e % (kBlk / 8));
      *reinterpret_cast<uint4 *>(dst + (vb * T_ + t) * kBlk + ch * 8) =
          *reinterpret_cast<const uint4 *>(src + (b * T_ + t) * W + sel * kBlk + ch * 8);
    }
  }
}

// dense[b][s][i*64 + r][j*64 + c] <-> blocks[((b*nd + i)*nk + j)][s][r][c]
template <typename T, bool kToBlocks>
__global__ void __launch_bounds__(256)
state_blocks_kernel(T *__restrict__ dense, T *__restrict__ blocks, int64_t B, int64_t S, int D, int K,
                    int nd, int nk) {
  const int64_t n = B * nd * nk * S * kBlk * (kBlk / 8);
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int ch = (int)(idx % (kBlk / 8));
    const int r = (int)((idx / (kBlk / 8)) % kBlk);
    const int64_t s = (idx / ((kBlk / 8) * kBlk)) % S;
    const int64_t vb = idx / ((int64_t)(kBlk / 8) * kBlk * S);
    const int j = (int)(vb % nk), i = (int)((vb / nk) % nd);
    const int64_t b = vb / ((int64_t)nk * nd);
    T *dp = dense + ((b * S + s) * D + i * kBlk + r) * K + j * kBlk + ch * 8;
    T *bp = blocks + ((vb * S + s) * kBlk + r) * kBlk + ch * 8;
    if (kToBlocks)
      *reinterpret_cast<uint4 *>(bp) = *reinterpret_cast<const uint4 *>(dp);
    else
      *reinterpret_cast<uint4 *>(dp) = *reinterpret_cast<const uint4 *>(bp);
  }
}

// dst[b][t][sel*64 + e] = sum over the other block index of src[((b*nd + i)*nk + j)][t][e];
// eight elements (16 bytes) per thread
template <typename T>
__global__ void __launch_bounds__(256)
combine_vec_kernel(const T *__restrict__ src, T *__restrict__ dst, int64_t B, int64_t T_, int W, int nd,
                   int nk, int dside) {
  const int nsel = dside ? nd : nk, nother = dside ? nk : nd;
  const int64_t n = B * T_ * nsel * (kBlk / 8);
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int e8 = (int)(idx % (kBlk / 8));
    const int sel = (int)((idx / (kBlk / 8)) % nsel);
    const int64_t t = (idx / ((int64_t)(kBlk / 8) * nsel)) % T_;
    const int64_t b = idx / ((int64_t)(kBlk / 8) * nsel * T_);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int o = 0; o < nother; ++o) {
      const int i = dside ? sel : o, j = dside ? o : sel;
      const int64_t vb = (b * nd + i) * nk + j;
      const uint4 u = *reinterpret_cast<const uint4 *>(src + (vb * T_ + t) * kBlk + 8 * e8);
      const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float2 v = Pair<T>::ld(e + 2 * r);
        acc[2 * r] += v.x;
        acc[2 * r + 1] += v.y;
      }
    }
    uint4 o4;
    T *oe = reinterpret_cast<T *>(&o4);
#pragma unroll
    for (int r = 0; r < 4; ++r) Pair<T>::st(oe + 2 * r, acc[2 * r], acc[2 * r + 1]);
    *reinterpret_cast<uint4 *>(dst + (b * T_ + t) * W + sel * kBlk + 8 * e8) = o4;
  }
}

inline unsigned grid_for(int64_t n_items) {
  const int64_t blocks = ceil_div64(n_items, 256);
  return (unsigned)(blocks < 148 * 16 ? (blocks < 1 ? 1 : blocks) : 148 * 16);
}

struct Layout {
  int64_t B, T_, D, K, nd, nk, VB, slots, ckpt_every;
  size_t esz;
  size_t vec() const { return (size_t)VB * T_ * kBlk * esz; }          // one virtual-batch vector tensor
  size_t st() const { return (size_t)VB * kBlk * kBlk * esz; }         // one virtual-batch state
  size_t ck() const { return (size_t)VB * slots * kBlk * kBlk * esz; } // virtual-batch checkpoints
};

Layout make_layout(int64_t B, int64_t T_, int64_t D, int64_t K, int64_t ckpt_every) {
  Layout l;
  l.B = B; l.T_ = T_; l.D = D; l.K = K;
  l.nd = D / kBlk; l.nk = K / kBlk; l.VB = B * l.nd * l.nk;
  l.slots = ceil_div64(T_, ckpt_every);
  l.ckpt_every = ckpt_every;
  l.esz = 2;
  return l;
}

size_t a256(size_t v) { return align_up(v, 256); }

// Copies of the flagged blocks' input windows for the scan kernels.
template <typename T>
void gather_flagged(const void *src, T *dst, const Layout &l, int W, int dside, const int *rowflag, cudaStream_t st) {
  const int64_t items = l.VB * kGatherSlices;
  gather_vec_kernel<T><<<(unsigned)(items < 148 * 8 ? items : 148 * 8), 256, 0, st>>>(
      (const T *)src, dst, l.B, l.T_, W, (int)l.nd, (int)l.nk, dside, rowflag);
}

template <typename T>
int blocked_forward_typed(const void *x, const void *f, const void *q, const void *k, const void *fk,
                          const void *state, void *out, void *ckpt, const Layout &l, void *scratch,
                          cudaStream_t st) {
  unsigned char *p = static_cast<unsigned char *>(scratch);
  auto take = [&](size_t bytes) { unsigned char *r = p; p += a256(bytes); return r; };
  T *xq = (T *)take(l.vec()), *fq = (T *)take(l.vec()), *qq = (T *)take(l.vec());
  T *kq = (T *)take(l.vec()), *fkq = (T *)take(l.vec()), *oq = (T *)take(l.vec());
  T *sq = (T *)take(l.st()), *cq = (T *)take(l.ck());
  void *inner = p;
  const int dt = std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16;
  const int nd = (int)l.nd, nk = (int)l.nk, D = (int)l.D, K = (int)l.K;
  state_blocks_kernel<T, true><<<grid_for(l.VB * kBlk * 8), 256, 0, st>>>(
      (T *)const_cast<void *>(state), sq, l.B, 1, D, K, nd, nk);
  T2FW_CHECK_LAUNCH(1);
  const int *rowflag = nullptr;
  int rc = lfw_chunk_forward_grid(x, f, q, k, fk, sq, oq, cq, l.B, l.T_, nd, nk, dt, l.ckpt_every, inner, st, &rowflag);
  if (rc != T2FW_OK) return rc;
  gather_flagged<T>(x, xq, l, D, 1, rowflag, st);
  gather_flagged<T>(f, fq, l, D, 1, rowflag, st);
  gather_flagged<T>(q, qq, l, K, 0, rowflag, st);
  gather_flagged<T>(k, kq, l, K, 0, rowflag, st);
  gather_flagged<T>(fk, fkq, l, K, 0, rowflag, st);
  T2FW_CHECK_LAUNCH(5);
  rc = lfw_scan_forward(xq, fq, qq, kq, fkq, sq, oq, cq, l.VB, l.T_, kBlk, kBlk, dt, l.ckpt_every, st, rowflag);
  if (rc != T2FW_OK) return rc;
  combine_vec_kernel<T><<<grid_for(l.B * l.T_ * l.nd * (kBlk / 8)), 256, 0, st>>>(
      oq, (T *)out, l.B, l.T_, D, nd, nk, 1);
  state_blocks_kernel<T, false><<<grid_for(l.VB * l.slots * kBlk * 8), 256, 0, st>>>(
      (T *)ckpt, cq, l.B, l.slots, D, K, nd, nk);
  T2FW_CHECK_LAUNCH(2);
  return T2FW_OK;
}

template <typename T>
int blocked_backward_typed(const void *go, const void *gs, const void *x, const void *f, const void *q,
                           const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
                           void *df, void *dq, void *dk, void *dfk, void *ds, const Layout &l,
                           void *scratch, cudaStream_t st) {
  unsigned char *p = static_cast<unsigned char *>(scratch);
  auto take = [&](size_t bytes) { unsigned char *r = p; p += a256(bytes); return r; };
  T *xq = (T *)take(l.vec()), *fq = (T *)take(l.vec()), *qq = (T *)take(l.vec());
  T *kq = (T *)take(l.vec()), *fkq = (T *)take(l.vec()), *goq = (T *)take(l.vec());
  T *dxq = (T *)take(l.vec()), *dfq = (T *)take(l.vec()), *dqq = (T *)take(l.vec());
  T *dkq = (T *)take(l.vec()), *dfkq = (T *)take(l.vec());
  T *sq = (T *)take(l.st()), *gsq = (T *)take(l.st()), *dsq = (T *)take(l.st()), *cq = (T *)take(l.ck());
  void *inner = p;
  const int dt = std::is_same<T, __half>::value ? T2FW_F16 : T2FW_BF16;
  const int nd = (int)l.nd, nk = (int)l.nk, D = (int)l.D, K = (int)l.K;
  state_blocks_kernel<T, true><<<grid_for(l.VB * kBlk * 8), 256, 0, st>>>(
      (T *)const_cast<void *>(state), sq, l.B, 1, D, K, nd, nk);
  state_blocks_kernel<T, true><<<grid_for(l.VB * kBlk * 8), 256, 0, st>>>(
      (T *)const_cast<void *>(gs), gsq, l.B, 1, D, K, nd, nk);
  state_blocks_kernel<T, true><<<grid_for(l.VB * l.slots * kBlk * 8), 256, 0, st>>>(
      (T *)const_cast<void *>(ckpt), cq, l.B, l.slots, D, K, nd, nk);
  T2FW_CHECK_LAUNCH(3);
  const int *rowflag = nullptr;
  int rc = lfw_chunk_backward_grid(go, gsq, x, f, q, k, fk, sq, cq, dxq, dfq, dqq, dkq, dfkq, dsq, l.B, l.T_, nd, nk,
                                   dt, l.ckpt_every, inner, st, &rowflag);
  if (rc != T2FW_OK) return rc;
  gather_flagged<T>(x, xq, l, D, 1, rowflag, st);
  gather_flagged<T>(f, fq, l, D, 1, rowflag, st);
  gather_flagged<T>(go, goq, l, D, 1, rowflag, st);
  gather_flagged<T>(q, qq, l, K, 0, rowflag, st);
  gather_flagged<T>(k, kq, l, K, 0, rowflag, st);
  gather_flagged<T>(fk, fkq, l, K, 0, rowflag, st);
  T2FW_CHECK_LAUNCH(6);
  rc = lfw_scan_backward(goq, gsq, xq, fq, qq, kq, fkq, sq, cq, dxq, dfq, dqq, dkq, dfkq, dsq, l.VB, l.T_,
                         kBlk, kBlk, dt, l.ckpt_every, st, rowflag);
  if (rc != T2FW_OK) return rc;
  const unsigned gd = grid_for(l.B * l.T_ * l.nd * (kBlk / 8)), gk = grid_for(l.B * l.T_ * l.nk * (kBlk / 8));
  combine_vec_kernel<T><<<gd, 256, 0, st>>>(dxq, (T *)dx, l.B, l.T_, D, nd, nk, 1);
  combine_vec_kernel<T><<<gd, 256, 0, st>>>(dfq, (T *)df, l.B, l.T_, D, nd, nk, 1);
  combine_vec_kernel<T><<<gk, 256, 0, st>>>(dqq, (T *)dq, l.B, l.T_, K, nd, nk, 0);
  combine_vec_kernel<T><<<gk, 256, 0, st>>>(dkq, (T *)dk, l.B, l.T_, K, nd, nk, 0);
  combine_vec_kernel<T><<<gk, 256, 0, st>>>(dfkq, (T *)dfk, l.B, l.T_, K, nd, nk, 0);
  state_blocks_kernel<T, false><<<grid_for(l.VB * kBlk * 8), 256, 0, st>>>((T *)ds, dsq, l.B, 1, D, K, nd, nk);
  T2FW_CHECK_LAUNCH(6);
  return T2FW_OK;
}

}  // namespace

bool lfw_blocked_supported(int64_t D, int64_t K, int dtype, int64_t ckpt_every) {
  if (dtype != T2FW_F16 && dtype != T2FW_BF16) return false;
  if (ckpt_every < kC || ckpt_every % kC != 0) return false;
  if (D % kBlk != 0 || K % kBlk != 0 || D > 256 || K > 256) return false;
  return D > kBlk || K > kBlk;
}

size_t lfw_blocked_forward_scratch_bytes(int64_t B, int64_t T_, int64_t D, int64_t K, int64_t ckpt_every) {
  const Layout l = make_layout(B, T_, D, K, ckpt_every);
  return 6 * a256(l.vec()) + a256(l.st()) + a256(l.ck()) + lfw_chunk_forward_scratch_bytes(l.VB, T_, ckpt_every);
}

size_t lfw_blocked_backward_scratch_bytes(int64_t B, int64_t T_, int64_t D, int64_t K, int64_t ckpt_every) {
  const Layout l = make_layout(B, T_, D, K, ckpt_every);
  return 11 * a256(l.vec()) + 3 * a256(l.st()) + a256(l.ck()) + lfw_chunk_backward_scratch_bytes(l.VB, T_, ckpt_every);
}

int lfw_blocked_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                        const void *state, void *out, void *ckpt, int64_t B, int64_t T_, int64_t D,
                        int64_t K, int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st) {
  const Layout l = make_layout(B, T_, D, K, ckpt_every);
  if (dtype == T2FW_F16)
    return blocked_forward_typed<__half>(x, f, q, k, fk, state, out, ckpt, l, scratch, st);
  return blocked_forward_typed<__nv_bfloat16>(x, f, q, k, fk, state, out, ckpt, l, scratch, st);
}

int lfw_blocked_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                         const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
                         void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B, int64_t T_,
                         int64_t D, int64_t K, int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st) {
  const Layout l = make_layout(B, T_, D, K, ckpt_every);
  if (dtype == T2FW_F16)
    return blocked_backward_typed<__half>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk, ds,
                                          l, scratch, st);
  return blocked_backward_typed<__nv_bfloat16>(go, gs, x, f, q, k, fk, state, ckpt, dx, df, dq, dk, dfk,
                                               ds, l, scratch, st);
}

}  // namespace t2fw
