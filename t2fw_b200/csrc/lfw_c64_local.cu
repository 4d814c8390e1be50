// Chunk-local state contributions of the decay rule on the tcgen05 tensor core (D = K = 64,
// 16-bit storage, chunks of 64 steps): the first phase of the chunked forward and backward, before
// the carry over the chunks.  Together with the carry it replaces the reference's sequential scans
// (t2fw/csrc/lfw_kernel.cu:18-59 and :61-102).
//
// Forward:  L_c[d][k] = sum_t (x_t[d] * prod_{j>t} f_j[d]) * (k_t[k] * prod_{j>t} fk_j[k])
//           the chunk's own contribution to the state at the chunk end (products run to the end
//           of the chunk: nothing is divided, and no factor exceeds the inputs for gates <= 1)
// Backward: G_c[d][k] = sum_s (dO_s[d] * prod_{j<=s} f_j[d]) * (q_s[k] * prod_{j<=s} fk_j[k])
//           the chunk's own contribution to the state gradient at the chunk start
// Both are one 64 x 64 x 64 contraction over the chunk's steps, plus the chunk's total decay
// vectors.  A chunk whose products exceed 2^100 is flagged (its batch row is redone by the scan
// kernels); products that underflow lose nothing.
//
// Persistent CTAs of 16 warps, two per SM.  The four raw 8 KB input blocks of a chunk arrive by
// bulk asynchronous copy into one of two buffers.  Thread (side, feature, 16-step quarter) forms
// the product of its quarter, then walks its steps with a running product that starts from the
// quarters between it and the anchoring end of the chunk.  The d-side values become the A operand
// in tensor memory (row = feature, stored in both lane sets), the k-side values a K-major
// shared-memory tile; one lane issues the sixteen MMAs (two interleaved 32-column halves); the fp32
// result leaves with 32-byte stores.
#include <mutex>

#include "lfw_c64.cuh"
#include "seq_layout.cuh"

namespace t2fw {

using namespace c64;


namespace {

constexpr int kThreadsL = 512;
constexpr int kCtasPerSmL = 2;
// shared-memory map (bytes from the 1024-byte aligned base)
constexpr int oTk = 0;                             // k-side tile [k][t]
constexpr int oQtL = oTk + kTile;                  // quarter products [2 sides][4][64]
constexpr int oRawL = oQtL + 2 * 4 * kDim * 4;     // [2 buffers] val_d, gate_d, val_k, gate_k
constexpr int kSmemL = oRawL + 2 * 4 * kRawBytes + 1024;
static_assert(oRawL % 128 == 0, "bulk-copy destination alignment");
static_assert(kCtasPerSmL * (kSmemL + 1024) <= 227 * 1024, "two CTAs per SM");

constexpr int cA = 0, cD = 64;                     // tensor-memory columns
constexpr int kTmemColsL = 128;

// kSuffix = true : value * (product of the gates AFTER the step, to the chunk end)   [forward]
// kSuffix = false: value * (product of the gates up to and including the step)       [backward]
template <typename T, bool kSuffix>
__global__ void __launch_bounds__(kThreadsL, kCtasPerSmL)
lfw_c64_local_kernel(const __grid_constant__ seq::Maps mp, float *__restrict__ M, float *__restrict__ Ac,
                     float *__restrict__ Gc, int *__restrict__ flags, int *__restrict__ status, int64_t T_,
                     int64_t nc, int64_t total) {
  extern __shared__ __align__(1024) unsigned char sm_raw[];
  unsigned char *sm = sm_raw + ((1024u - (umma::smem_u32(sm_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t barRaw[2], barM;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail, s_bad;

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  // warps 0-7: d side, tensor-memory rows: lane quarter q4, column part, lane set h, row fl;
  //            thread = feature 16 * q4 + fl, quarter 2 * h + part of the chunk
  // warps 8-15: k side: thread = feature, quarter
  const bool dside = warp < 8;
  const int q4 = warp & 3, part = (warp >> 2) & 1, h = lane >> 4, fl = lane & 15;
  const int feat = dside ? 16 * q4 + fl : ((warp - 8) & 1) * 32 + lane;
  const int tq = dside ? 2 * h + part : (warp - 8) >> 1;
  float *qtot = reinterpret_cast<float *>(sm + oQtL);

  // tensors: 0 val_d, 1 gate_d, 2 val_k, 3 gate_k
  const bool unit_forget = (mp.flags & seq::kUnitForget) != 0;
  auto issue_raw = [&](int64_t ci, int buf) {     // thread 0 only: one copy per tensor
    const Item w = split_item(ci, nc, mp.heads);
    const int row = (int)(w.b * T_ + w.c * kC), hc = w.h;
    const int nv = (int)((T_ - (int64_t)w.c * kC < kC) ? T_ - (int64_t)w.c * kC : kC);
    unsigned char *r = sm + oRawL + buf * 4 * kRawBytes;
    const uint32_t per = (mp.flags & seq::kContiguous) ? (uint32_t)nv * kDim * sizeof(T) : (uint32_t)kRawBytes;
    acp::mbar_expect_tx(&barRaw[buf], (unit_forget ? 3u : 4u) * per);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (!(i == 1 && unit_forget)) seq::fetch_block<T>(mp, i, r + i * kRawBytes, row, hc, nv, &barRaw[buf]);
  };

  if (tid == 0) {
    umma::mbar_init(&barRaw[0], 1);
    umma::mbar_init(&barRaw[1], 1);
    umma::mbar_init(&barM, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, kTmemColsL);
  if (unit_forget) {      // the d-side gate block of both buffers is the constant 1 and never loaded
    seq::fill_block(reinterpret_cast<T *>(sm + oRawL + kRawBytes), 1.f, tid, kThreadsL);
    seq::fill_block(reinterpret_cast<T *>(sm + oRawL + 5 * kRawBytes), 1.f, tid, kThreadsL);
  }
  sync_all();
  dependency_wait();
  const uint32_t tb = __shfl_sync(0xffffffffu, tmem_slot, 0);
  const uint32_t tl = umma::tmem_addr(tb, 32 * q4, 0);
  uint32_t n_issued[2] = {0u, 0u}, n_landed[2] = {0u, 0u};      // thread 0: bulk-copy rounds per buffer
  if (tid == 0 && (int64_t)blockIdx.x < total) {
    issue_raw(blockIdx.x, 0);
    ++n_issued[0];
  }
  const uint64_t dTk = desc_sw128(umma::smem_u32(sm + oTk));

  uint32_t it = 0;
  for (int64_t ci = blockIdx.x; ci < total; ci += gridDim.x, ++it) {
    const int buf = it & 1;
    const int64_t c = (int64_t)((uint32_t)ci % (uint32_t)nc), t0c = c * kC;
    const int nvalid = (int)((T_ - t0c < kC) ? T_ - t0c : kC);
    T *raw = reinterpret_cast<T *>(sm + oRawL + buf * 4 * kRawBytes);
    if (tid == 0) {
      s_bad = 0;
      if (ci + gridDim.x < total) {      // the other buffer was released at the end of the previous chunk
        issue_raw(ci + gridDim.x, buf ^ 1);
        ++n_issued[buf ^ 1];
      }
    }
    if (acp::mbar_wait(&barRaw[buf], (it >> 1) & 1u)) {
      if (tid == 0) ++n_landed[buf];
    } else {
      s_fail = 1;
    }
    __syncthreads();
    if (s_fail) break;
    if ((mp.flags & seq::kSigmoidGate) || mp.q_scale != 1.f) {      // fused layer: activations applied here
      if (mp.flags & seq::kSigmoidGate) seq::sigmoid_gate_block(raw + 3 * kC * kDim, tid, kThreadsL);
      if (mp.q_scale != 1.f) seq::scale_block(raw + 2 * kC * kDim, mp.q_scale, tid, kThreadsL);
      __syncthreads();
    }
    if (nvalid < kC) {      // partial chunk: identity steps beyond the valid ones
      pad_raw_tail<T>(raw, 4, (1u << 1) | (1u << 3), nvalid, tid, kThreadsL);
      __syncthreads();
    }

    // ---- products of the four quarters ----
    const T *gcol = raw + (dside ? 1 : 3) * kC * kDim + feat, *vcol = raw + (dside ? 0 : 2) * kC * kDim + feat;
    float g[16];
    qtot[((dside ? 0 : 4) + tq) * kDim + feat] = load_gates16<T>(gcol, tq, g);
    __syncthreads();

    // ---- running products from the anchoring end, scaled values ----
    float w[16];
    {
      const float *qt = qtot + (dside ? 0 : 4) * kDim + feat;
      float s = 1.f, hi = 0.f;
      if (kSuffix) {
#pragma unroll
        for (int i = 3; i > 0; --i)
          if (i > tq) s *= qt[i * kDim];
#pragma unroll
        for (int j = 15; j >= 0; --j) {
          w[j] = bias_tf32(Elem<T>::ld(vcol + (16 * tq + j) * kDim) * s);
          s *= g[j];
          hi = fmaxf(hi, fabsf(s));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 3; ++i)
          if (i < tq) s *= qt[i * kDim];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          s *= g[j];
          hi = fmaxf(hi, fabsf(s));
          w[j] = bias_tf32(Elem<T>::ld(vcol + (16 * tq + j) * kDim) * s);
        }
      }
      if (!(hi <= kRangeHi)) s_bad = 1;     // also catches NaN
      // total decay of the chunk for this feature
      if (tq == (kSuffix ? 0 : 3)) (dside ? Ac : Gc)[(size_t)ci * kDim + feat] = s;
    }
    if (dside) {
      // A operand [d][t] in both lane sets: the lower half warp holds quarter `part`, the upper
      // half warp quarter 2 + part of the same rows; one store names one column range per warp
      float lo[16], hi2[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float p = __shfl_xor_sync(0xffffffffu, w[j], 16);
        lo[j] = h ? p : w[j];
        hi2[j] = h ? w[j] : p;
      }
      umma::tmem_st16(tl + cA + 16 * part, lo);
      umma::tmem_st16(tl + cA + 32 + 16 * part, hi2);
      umma::tmem_st_wait();
    } else {
      unsigned char *tk = sm + oTk;
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4 *>(tk + toff(feat, 16 * tq + j)) = make_float4(w[j], w[j + 1], w[j + 2], w[j + 3]);
    }
    umma::fence_async_smem();
    sync_all();       // operands complete, raw buffer consumed

    if (warp == 0) {
      const uint32_t d0 = tb, d1 = umma::tmem_addr(tb, 16, 0);
      constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
      constexpr uint64_t n1 = (uint64_t)(32 * 128 >> 4);     // k rows 32..63
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
          mma_tf32_ts(d0 + cD, d0 + cA + 8 * ks, dTk + o, idesc, ks > 0);
          mma_tf32_ts(d1 + cD, d1 + cA + 8 * ks, dTk + n1 + o, idesc, ks > 0);
        }
        umma::mma_commit(&barM);
      }
      __syncwarp();
      if (tid == 0) flags[ci] = s_bad;
    }
    if (!umma::mbar_wait(&barM, it & 1u)) {
      s_fail = 1;
      flags[ci] = 1;      // results unusable: let the scan kernels redo the row
    }
    umma::fence_after_sync();
    {
      // thread (lane quarter, column part, lane set, row): row d, columns 32 * h + 8 * (warp >> 2) .. + 7
      const int d = 16 * q4 + fl, k0 = 32 * h + 8 * (warp >> 2);
      float v[8];
      umma::tmem_ld8(tl + cD + 8 * (warp >> 2), v);
      umma::tmem_ld_wait();
      float *dst = M + ((size_t)ci * kDim + d) * kDim + k0;
      *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    // No barrier here: the next chunk writes nothing before the barrier at its start, which every
    // thread reaches only after this read-out; that barrier also spreads s_fail.
    umma::fence_before_sync();
  }
  __syncthreads();      // s_fail of the last chunk is visible
  if (tid == 0) {
    if (s_fail) atomicExch(status, 1);
    for (int bb = 0; bb < 2; ++bb)     // bounded: let copies that are still in flight land
      if (n_issued[bb] > n_landed[bb]) acp::mbar_wait(&barRaw[bb], n_landed[bb] & 1u);
  }
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, kTmemColsL);
}

}  // namespace

__device__ int g_umma_status = 0;

namespace {
int *g_umma_status_addr[64] = {};
int g_sm_count[64] = {};
std::mutex g_status_mutex;
}

// device address of the status word kernels set when a bounded wait expires
int lfw_chunk_status_ptr(int **out) {
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("device index %d out of range", dev);
    return T2FW_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_umma_status_addr[dev] == nullptr) {
    int n = 0;
    T2FW_CHECK_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    void *p = nullptr;
    T2FW_CHECK_CUDA(cudaGetSymbolAddress(&p, g_umma_status));
    g_sm_count[dev] = n;                               // filled before the address is published
    g_umma_status_addr[dev] = static_cast<int *>(p);
  }
  *out = g_umma_status_addr[dev];
  return T2FW_OK;
}

// number of SMs of the current device (cached with the status address)
int lfw_chunk_sm_count(int *out) {
  int *unused = nullptr;
  const int rc = lfw_chunk_status_ptr(&unused);
  if (rc != T2FW_OK) return rc;
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  *out = g_sm_count[dev];
  return T2FW_OK;
}

int lfw_chunk_umma_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// Forward flavour: M = L_c from (x, f) and (k, fk).  Backward flavour: M = G_c from (dO, f), (q, fk).
// mp describes the four tensors in that order (mp.q_scale applies to the third one).
int lfw_chunk_local_umma(bool backward, const seq::Maps &mp, float *M, float *Ac, float *Gc, int *flags, int64_t BH,
                         int64_t T_, int dtype, cudaStream_t st) {
  const int64_t nc = ceil_div64(T_, kC), total = BH * nc;
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  int sms = 0;
  rc = lfw_chunk_sm_count(&sms);
  if (rc != T2FW_OK) return rc;
  const int64_t max_ctas = (int64_t)sms * kCtasPerSmL;
  const unsigned grid = (unsigned)(total < max_ctas ? total : max_ctas);
#define T2FW_LAUNCH(TT, SUF)                                                                          \
  do {                                                                                                \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_c64_local_kernel<TT, SUF>,                               \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemL));       \
    T2FW_CHECK_CUDA(launch_dependent(lfw_c64_local_kernel<TT, SUF>, dim3(grid), dim3(kThreadsL), kSmemL, st, mp, M, \
                                     Ac, Gc, flags, status, T_, nc, total));                         \
  } while (0)
  if (dtype == T2FW_F16) {
    if (backward) T2FW_LAUNCH(__half, false); else T2FW_LAUNCH(__half, true);
  } else {
    if (backward) T2FW_LAUNCH(__nv_bfloat16, false); else T2FW_LAUNCH(__nv_bfloat16, true);
  }
#undef T2FW_LAUNCH
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw

