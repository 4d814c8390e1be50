// Chunk-local state contributions of the decay rule on the tcgen05 tensor core (D = K = 64).
//
// Forward:  L_c[d][k] = sum_{t in chunk} (x_t[d] * prod_{j>t} f_j[d]) * (k_t[k] * prod_{j>t} fk_j[k])
//           the chunk's own contribution to the state at the chunk end (products run to the end
//           of the chunk, so nothing is divided and no factor exceeds the inputs for gates <= 1)
// Backward: G_c[d][k] = sum_{s in chunk} (dO_s[d] * prod_{j<=s} f_j[d]) * (q_s[k] * prod_{j<=s} fk_j[k])
//           the chunk's own contribution to the state gradient at the chunk start
// Both are one 64 x 64 x 64 contraction over the chunk's time steps.
//
// The kernel is persistent.  Per chunk: the four raw 8 KB input blocks arrive by bulk
// asynchronous copy (prefetched while the previous chunk is processed); each thread owns one
// feature column, walks the 64 steps with a running gate product and writes its scaled values
// as one row of a K-major TF32 operand tile in shared memory; one thread issues the
// tcgen05.mma instructions (two N = 32 halves into the two interleaved lane sets of tensor
// memory); everyone waits on an mbarrier with a bounded spin; the accumulators are read back
// with tcgen05.ld and stored as fp32.  The mma.sync kernels lfw_chunk_local_kernel /
// lfw_chunk_bwd_local_kernel write the same scratch layout and remain as the fallback.
#include "async_copy.cuh"
#include "lfw_chunk.cuh"
#include "umma.cuh"

namespace t2fw {

using namespace chunk;

namespace {

constexpr int kTileBytes = umma::tile_bytes(kDim, kC);   // [64 features][64 steps] fp32, interleaved
constexpr int kRawVec = kC * kDim;                        // elements of one raw input block
constexpr int kCtasPerSm = 3;

// kSuffix = true : value * (product of the gates AFTER the step, to the chunk end)   [forward]
// kSuffix = false: value * (product of the gates up to and including the step)       [backward]
template <typename T, bool kSuffix>
__global__ void __launch_bounds__(kThreads)
lfw_chunk_local_umma_kernel(const T *__restrict__ val_d, const T *__restrict__ gate_d,
                            const T *__restrict__ val_k, const T *__restrict__ gate_k,
                            float *__restrict__ M, float *__restrict__ Ac, float *__restrict__ Gc,
                            int *__restrict__ flags, int *__restrict__ status, int64_t T_, int64_t nc,
                            int64_t total) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar_mma, bar_raw;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_flag, s_fail;
  unsigned char *tA = smem, *tB = smem + kTileBytes;   // A: d side, B: k side
  T *r_vd = reinterpret_cast<T *>(smem + 2 * kTileBytes), *r_gd = r_vd + kRawVec;
  T *r_vk = r_gd + kRawVec, *r_gk = r_vk + kRawVec;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto issue = [&](int64_t ci) {     // thread 0 only
    const int64_t b = ci / nc, c = ci % nc, t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const uint32_t vb = (uint32_t)nv * kDim * sizeof(T);
    const size_t base = ((size_t)b * T_ + t0) * kDim;
    acp::mbar_expect_tx(&bar_raw, 4 * vb);
    acp::bulk_g2s(r_vd, val_d + base, vb, &bar_raw);
    acp::bulk_g2s(r_gd, gate_d + base, vb, &bar_raw);
    acp::bulk_g2s(r_vk, val_k + base, vb, &bar_raw);
    acp::bulk_g2s(r_gk, gate_k + base, vb, &bar_raw);
  };

  if (threadIdx.x == 0) {
    umma::mbar_init(&bar_mma, 1);
    umma::mbar_init(&bar_raw, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 32);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tbase = tmem_slot;
  if (threadIdx.x == 0 && (int64_t)blockIdx.x < total) issue(blockIdx.x);

  const bool kside = threadIdx.x < kDim;
  const int col = kside ? threadIdx.x : threadIdx.x - kDim;
  const T *gp = (kside ? r_gk : r_gd) + col;
  const T *vp = (kside ? r_vk : r_vd) + col;
  unsigned char *tile = kside ? tB : tA;

  uint32_t it = 0;
  for (int64_t ci = blockIdx.x; ci < total; ci += gridDim.x, ++it) {
    const int64_t b = ci / nc, c = ci % nc;
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    if (threadIdx.x == 0) s_flag = 0;
    if (!acp::mbar_wait(&bar_raw, it & 1u)) s_fail = 1;   // benign race: every writer stores 1
    __syncthreads();
    if (s_fail) break;

    // ---- operand tiles: thread = one feature column, 64 steps with a running gate product --
    {
      float p = 1.f;                         // running product over the chunk
      float pb = 1.f, lo = 1.f, hi = 1.f;    // running product inside the current 16-step block
      bool bad = false;
      float buf[4];
#pragma unroll 16
      for (int tt = 0; tt < kC; ++tt) {
        const int t = kSuffix ? kC - 1 - tt : tt;
        const bool in = t < nvalid;
        const float g = sanitize_gate(in ? Elem<T>::ld(gp + t * kDim) : 1.f);
        const float v = in ? Elem<T>::ld(vp + t * kDim) : 0.f;
        float w;
        if (kSuffix) {
          w = v * p;
          p *= g;
        } else {
          p *= g;
          w = v * p;
        }
        pb *= g;
        lo = fminf(lo, fabsf(pb));
        hi = fmaxf(hi, fabsf(pb));
        if ((tt & (kSub - 1)) == kSub - 1) {
          // every product of consecutive gates inside the block lies in [lo/hi, hi/lo]
          bad |= !(hi <= lo * kRangeHi);
          pb = 1.f; lo = 1.f; hi = 1.f;
        }
        bad |= !(fabsf(p) <= kRangeHi);
        buf[t & 3] = round_tf32(w);
        if ((kSuffix && (t & 3) == 0) || (!kSuffix && (t & 3) == 3))
          *reinterpret_cast<float4 *>(tile + umma::tile_off(col, t & ~3, kC)) =
              make_float4(buf[0], buf[1], buf[2], buf[3]);
      }
      if (bad) s_flag = 1;
      (kside ? Gc : Ac)[(size_t)ci * kDim + col] = p;   // total decay of the chunk for this column
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();            // tiles complete, raw blocks consumed
    umma::fence_after_sync();

    if (threadIdx.x == 0) {
      if (ci + gridDim.x < total) issue(ci + gridDim.x);   // prefetch the next chunk's inputs
      const uint32_t idesc = umma::make_idesc_tf32(kDim, 32, false, false);
      const uint32_t ta = umma::smem_u32(tA), tb = umma::smem_u32(tB);
#pragma unroll
      for (int h = 0; h < 2; ++h) {            // k columns 32h .. 32h+31 -> lane set h
        const uint32_t d = umma::tmem_addr(tbase, 16 * h, 0);
#pragma unroll
        for (int ks = 0; ks < kC / 8; ++ks)
          umma::mma_tf32(d, umma::desc_kmajor(ta, kC, 0, ks), umma::desc_kmajor(tb, kC, 32 * h, ks), idesc,
                         ks > 0);
      }
      umma::mma_commit(&bar_mma);
      flags[ci] = s_flag;
    }
    if (!umma::mbar_wait(&bar_mma, it & 1u)) s_fail = 1;
    __syncthreads();
    umma::fence_after_sync();
    if (s_fail) {
      if (threadIdx.x == 0) flags[ci] = 1;   // results unusable: let the scan kernels redo the row
      break;
    }
    {
      // lanes 0-15: rows 16w.., columns 0-31;  lanes 16-31: the same rows, columns 32-63
      const int row = 16 * warp + (lane & 15), c0 = 32 * (lane >> 4);
      float *dst = M + ((size_t)ci * kDim + row) * kDim + c0;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float v[16];
        umma::tmem_ld16(umma::tmem_addr(tbase, 32 * warp, 16 * j), v);
        umma::tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; e += 4)
          *reinterpret_cast<float4 *>(dst + 16 * j + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
      }
    }
    umma::fence_before_sync();   // accumulator reads are ordered before the next chunk's MMAs
  }
  if (s_fail && threadIdx.x == 0) atomicExch(status, 1);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tbase, 32);
}

}  // namespace

__device__ int g_umma_status = 0;

namespace {
int *g_umma_status_addr[64] = {};
int g_sm_count[64] = {};
}

// device address of the status word kernels set when a bounded wait expires
int lfw_chunk_status_ptr(int **out) {
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("device index %d out of range", dev);
    return T2FW_ERR_UNSUPPORTED;
  }
  if (g_umma_status_addr[dev] == nullptr) {
    void *p = nullptr;
    T2FW_CHECK_CUDA(cudaGetSymbolAddress(&p, g_umma_status));
    g_umma_status_addr[dev] = static_cast<int *>(p);
    T2FW_CHECK_CUDA(cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
  }
  *out = g_umma_status_addr[dev];
  return T2FW_OK;
}

int lfw_chunk_umma_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Forward flavour: M = L_c from (x, f) and (k, fk).  Backward flavour: M = G_c from (dO, f), (q, fk).
// Returns T2FW_ERR_UNSUPPORTED without launching if a pointer is not 16-byte aligned.
int lfw_chunk_local_umma(bool backward, const void *val_d, const void *gate_d, const void *val_k,
                         const void *gate_k, float *M, float *Ac, float *Gc, int *flags, int64_t B,
                         int64_t T_, int dtype, cudaStream_t st) {
  if (!(aligned16(val_d) && aligned16(gate_d) && aligned16(val_k) && aligned16(gate_k) && aligned16(M)))
    return T2FW_ERR_UNSUPPORTED;
  const int64_t nc = ceil_div64(T_, kC), total = B * nc;
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  const int64_t max_ctas = (int64_t)g_sm_count[dev] * kCtasPerSm;
  const size_t smem = 2 * (size_t)kTileBytes + 4 * (size_t)kRawVec * 2;
  const unsigned grid = (unsigned)(total < max_ctas ? total : max_ctas);
#define T2FW_LAUNCH(TT, SUF)                                                                          \
  do {                                                                                                \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_chunk_local_umma_kernel<TT, SUF>,                        \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
    lfw_chunk_local_umma_kernel<TT, SUF><<<grid, kThreads, smem, st>>>(                               \
        (const TT *)val_d, (const TT *)gate_d, (const TT *)val_k, (const TT *)gate_k, M, Ac, Gc, flags, \
        status, T_, nc, total);                                                                       \
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
