// Delta rule, chunked forward with the per-chunk products on the tcgen05 tensor core
// (D = M = 64, 16-bit storage).  Same mathematics and interface as dfw_chunk_fwd_kernel in
// dfw_chunk.cu (which stays as the mma.sync fallback):
//   Dl = U - W S^T ,  O = Q S^T + strict_lower(Q K^T) Dl ,  S += Dl^T K        per chunk of 64 steps
// One CTA per batch row walks the chunks in order.  Operands are TF32 tiles in the un-swizzled
// core-matrix layout, all K-major (tile rows = M / N index, contraction along tile columns), so
// K and Dl are also kept transposed.  Accumulators live in tensor memory as M = 64 tiles, two per
// column range (lane sets A = lanes 0-15 and B = lanes 16-31 of every lane quarter):
//   columns  0-63 :  A: W S^T            B: Q K^T
//   columns 64-127:  A: S (persistent)   B: Q S^T, then O (the second round accumulates onto it)
// (a tensor-memory load names one column range for the whole warp, so the two results that are
// read together share their columns)
// so the state never leaves tensor memory between chunks; after each chunk it is read once to
// refresh its TF32 copy in shared memory.  The two halves of every warp work on the two lane sets.
// The raw inputs of the next chunk arrive by bulk asynchronous copies while the current chunk is
// processed; every wait is bounded.
#include <type_traits>

#include "async_copy.cuh"
#include "lfw_chunk.cuh"
#include "umma.cuh"

namespace t2fw {

using namespace chunk;

int lfw_chunk_status_ptr(int **out);   // lfw_chunk_local_umma.cu

#ifdef T2FW_DFW_PROFILE
__device__ long long g_dfw_prof[16];
#define PROF(i)                                                    \
  do {                                                             \
    if (threadIdx.x == 0 && blockIdx.x == 0) {                     \
      const long long now_ = clock64();                            \
      g_dfw_prof[i] += now_ - tprev;                               \
      tprev = now_;                                                \
    }                                                              \
  } while (0)
#else
#define PROF(i)
#endif

namespace {

constexpr int kTh = 256;                                  // 4 lane quarters x 2 column halves
constexpr int kTileU = umma::tile_bytes(kDim, kC);        // 18432: [64][64] TF32, core-matrix layout
constexpr int oQ = 0, oK = kTileU, oKT = 2 * kTileU, oW = 3 * kTileU, oSt = 4 * kTileU, oAs = 5 * kTileU,
              oDT = 6 * kTileU;
constexpr int oRawQ = 7 * kTileU;                         // 16-bit [64][64]
constexpr int oRawK = oRawQ + kC * kDim * 2;
constexpr int oRawW = oRawK + kC * kDim * 2;              // fp32 [64][64]
constexpr int oRawU = oRawW + kC * kDim * 4;
constexpr int kSmemU = oRawU + kC * kDim * 4;
static_assert(kSmemU <= 227 * 1024 && oRawQ % 128 == 0, "shared memory layout");
constexpr int cWS = 0, cSt = 64;                          // tensor-memory columns (both lane sets)

__device__ __forceinline__ void sync_all() {
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
}

template <typename T>
__global__ void __launch_bounds__(kTh, 1)
dfw_chunk_fwd_umma_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ state,
                          const float *__restrict__ W, const float *__restrict__ U, T *__restrict__ out,
                          T *__restrict__ final_state, float *__restrict__ delta, int *__restrict__ status,
                          int64_t T_, int64_t nc) {
  extern __shared__ __align__(128) unsigned char sm[];
  __shared__ __align__(8) uint64_t bar_mma, bar_raw;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;

  const int64_t b = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3, half = warp >> 2, side = lane >> 4, fl = lane & 15;
  const int row = 16 * qd + fl, c0 = 32 * half;
  float *tQ = reinterpret_cast<float *>(sm + oQ);
  unsigned char *tS = sm + oSt;

  auto issue_raw = [&](int64_t c) {     // thread 0 only
    const int64_t t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const uint32_t vb = (uint32_t)nv * kDim * sizeof(T);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = ((size_t)b * nc + c) * kC * kDim;
    acp::mbar_expect_tx(&bar_raw, 2 * vb + 2 * kC * kDim * 4);
    acp::bulk_g2s(sm + oRawQ, q + base, vb, &bar_raw);
    acp::bulk_g2s(sm + oRawK, k + base, vb, &bar_raw);
    acp::bulk_g2s(sm + oRawW, W + tile, kC * kDim * 4, &bar_raw);
    acp::bulk_g2s(sm + oRawU, U + tile, kC * kDim * 4, &bar_raw);
  };

  if (tid == 0) {
    umma::mbar_init(&bar_mma, 1);
    umma::mbar_init(&bar_raw, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);
  sync_all();
  const uint32_t tb = tmem_slot;
  const uint32_t tl = umma::tmem_addr(tb, 32 * qd, 0);
  if (tid == 0) issue_raw(0);

  // initial state: row `row`, columns c0 .. c0+31 -> tensor memory (lane set A) and the TF32 tile
  {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = 0.f;
    if (side == 0) {
      const T *sp = state + (size_t)b * kDim * kDim + row * kDim + c0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float2 p = Pair<T>::ld(sp + 2 * j);
        v[2 * j] = p.x;
        v[2 * j + 1] = p.y;
      }
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4 *>(tS + umma::tile_off(row, c0 + j, kDim)) =
            make_float4(round_tf32(v[j]), round_tf32(v[j + 1]), round_tf32(v[j + 2]), round_tf32(v[j + 3]));
    }
    umma::tmem_st16(tl + cSt + c0, v);            // lanes B receive zeros (overwritten by Q S^T)
    umma::tmem_st16(tl + cSt + c0 + 16, v + 16);
    umma::tmem_st_wait();
  }

  uint32_t p_mma = 0, p_raw = 0;
  auto wait_mma = [&]() {
    if (!s_fail && !umma::mbar_wait(&bar_mma, p_mma)) s_fail = 1;
    p_mma ^= 1u;
    umma::fence_after_sync();
  };

#ifdef T2FW_DFW_PROFILE
  long long tprev = clock64();
#endif
  for (int64_t c = 0; c < nc; ++c) {
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim;
    PROF(0);
    if (!s_fail && !acp::mbar_wait(&bar_raw, p_raw)) s_fail = 1;
    p_raw ^= 1u;
    __syncthreads();
    if (s_fail) break;
    PROF(1);

    // ---- raw blocks -> TF32 tiles: pieces of 4 consecutive columns, 1024 per block ----------------
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;
      const bool in = r < nvalid;
      const uint2 uq = in ? *reinterpret_cast<const uint2 *>(sm + oRawQ + (r * kDim + c4) * 2) : make_uint2(0u, 0u);
      const uint2 uk = in ? *reinterpret_cast<const uint2 *>(sm + oRawK + (r * kDim + c4) * 2) : make_uint2(0u, 0u);
      const float2 q0 = Pair<T>::ld(reinterpret_cast<const T *>(&uq.x)), q1 = Pair<T>::ld(reinterpret_cast<const T *>(&uq.y));
      const float2 k0 = Pair<T>::ld(reinterpret_cast<const T *>(&uk.x)), k1 = Pair<T>::ld(reinterpret_cast<const T *>(&uk.y));
      *reinterpret_cast<float4 *>(sm + oQ + umma::tile_off(r, c4, kDim)) = make_float4(q0.x, q0.y, q1.x, q1.y);
      *reinterpret_cast<float4 *>(sm + oK + umma::tile_off(r, c4, kDim)) = make_float4(k0.x, k0.y, k1.x, k1.y);
      // K^T[m][t] = K[t][m]
      *reinterpret_cast<float *>(sm + oKT + umma::tile_off(c4, r, kC)) = k0.x;
      *reinterpret_cast<float *>(sm + oKT + umma::tile_off(c4 + 1, r, kC)) = k0.y;
      *reinterpret_cast<float *>(sm + oKT + umma::tile_off(c4 + 2, r, kC)) = k1.x;
      *reinterpret_cast<float *>(sm + oKT + umma::tile_off(c4 + 3, r, kC)) = k1.y;
      const float4 w4 = *reinterpret_cast<const float4 *>(sm + oRawW + (r * kDim + c4) * 4);
      *reinterpret_cast<float4 *>(sm + oW + umma::tile_off(r, c4, kDim)) =
          make_float4(round_tf32(w4.x), round_tf32(w4.y), round_tf32(w4.z), round_tf32(w4.w));
    }
    // this thread's part of U (lane set A threads): row `row`, columns c0 .. c0+31
    float uv[32];
    if (side == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 u4 = *reinterpret_cast<const float4 *>(sm + oRawU + (row * kDim + c0 + j) * 4);
        uv[j] = u4.x; uv[j + 1] = u4.y; uv[j + 2] = u4.z; uv[j + 3] = u4.w;
      }
    }
    PROF(2);
    umma::fence_async_smem();
    sync_all();                       // tiles complete (the S tile since the end of the last chunk)
    PROF(3);

    if (tid == 0) {
      if (c + 1 < nc) issue_raw(c + 1);
      const uint32_t idesc = umma::make_idesc_tf32(kDim, kDim, false, false);
      const uint32_t aQ = umma::smem_u32(sm + oQ), aK = umma::smem_u32(sm + oK), aW = umma::smem_u32(sm + oW),
                     aS = umma::smem_u32(sm + oSt);
#pragma unroll
      for (int ks = 0; ks < kC / 8; ++ks) {
        umma::mma_tf32(umma::tmem_addr(tb, 0, cWS), umma::desc_kmajor(aW, kDim, 0, ks),
                       umma::desc_kmajor(aS, kDim, 0, ks), idesc, ks > 0);     // W S^T
        umma::mma_tf32(umma::tmem_addr(tb, 16, cSt), umma::desc_kmajor(aQ, kDim, 0, ks),
                       umma::desc_kmajor(aS, kDim, 0, ks), idesc, ks > 0);     // Q S^T
        umma::mma_tf32(umma::tmem_addr(tb, 16, cWS), umma::desc_kmajor(aQ, kDim, 0, ks),
                       umma::desc_kmajor(aK, kDim, 0, ks), idesc, ks > 0);     // Q K^T
      }
      umma::mma_commit(&bar_mma);
    }
    PROF(4);
    wait_mma();
    PROF(5);
    {
      // lane set A: Dl = U - W S^T (row t = `row`, columns d);  lane set B: scores (row t, columns i)
      float v[32];
      umma::tmem_ld16(tl + cWS + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + cWS + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      if (side == 0) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = uv[j] - v[j];
        if (row < nvalid) {
          float *dp = delta + base + (size_t)row * kDim + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(dp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)      // Dl^T[d][t]
          *reinterpret_cast<float *>(sm + oDT + umma::tile_off(c0 + j, row, kC)) = round_tf32(v[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j < row) ? round_tf32(v[j]) : 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(sm + oAs + umma::tile_off(row, c0 + j, kC)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    }
    PROF(6);
    umma::fence_async_smem();
    sync_all();
    PROF(7);
    if (tid == 0) {
      const uint32_t idesc = umma::make_idesc_tf32(kDim, kDim, false, false);
      const uint32_t aA = umma::smem_u32(sm + oAs), aD = umma::smem_u32(sm + oDT), aKT = umma::smem_u32(sm + oKT);
#pragma unroll
      for (int ks = 0; ks < kC / 8; ++ks) {
        umma::mma_tf32(umma::tmem_addr(tb, 16, cSt), umma::desc_kmajor(aA, kC, 0, ks),
                       umma::desc_kmajor(aD, kC, 0, ks), idesc, true);        // O += A Dl
        umma::mma_tf32(umma::tmem_addr(tb, 0, cSt), umma::desc_kmajor(aD, kC, 0, ks),
                       umma::desc_kmajor(aKT, kC, 0, ks), idesc, true);       // S += Dl^T K
      }
      umma::mma_commit(&bar_mma);
    }
    PROF(8);
    wait_mma();
    PROF(9);
    {
      // lane set B: O (row t, columns d) -> global;  lane set A: S (row d, columns m) -> TF32 tile
      float v[32];
      umma::tmem_ld16(tl + cSt + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + cSt + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      if (side) {
        if (row < nvalid) {
          T *op = out + base + (size_t)row * kDim + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 2) Pair<T>::st(op + j, v[j], v[j + 1]);
        }
      } else if (c + 1 < nc) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(tS + umma::tile_off(row, c0 + j, kDim)) =
              make_float4(round_tf32(v[j]), round_tf32(v[j + 1]), round_tf32(v[j + 2]), round_tf32(v[j + 3]));
      } else {
        T *fp = final_state + (size_t)b * kDim * kDim + row * kDim + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 2) Pair<T>::st(fp + j, v[j], v[j + 1]);
      }
    }
    umma::fence_before_sync();   // accumulator reads are ordered before the next chunk's MMAs
    PROF(10);
  }
  (void)tQ;
  if (s_fail && tid == 0) atomicExch(status, 1);
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, 128);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// returns T2FW_ERR_UNSUPPORTED (without launching) if a pointer is not 16-byte aligned
int dfw_chunk_forward_umma(const void *q, const void *k, const void *state, const float *W, const float *U,
                           void *out, void *final_state, void *delta, int64_t B, int64_t T_, int dtype,
                           cudaStream_t st) {
  if (!(aligned16(q) && aligned16(k) && aligned16(state) && aligned16(W) && aligned16(U) && aligned16(out) &&
        aligned16(final_state) && aligned16(delta)))
    return T2FW_ERR_UNSUPPORTED;
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  const int64_t nc = ceil_div64(T_, kC);
#define T2FW_LAUNCH(TT)                                                                                  \
  do {                                                                                                   \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_fwd_umma_kernel<TT>,                                  \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemU));          \
    dfw_chunk_fwd_umma_kernel<TT><<<(unsigned)B, kTh, kSmemU, st>>>(                                     \
        (const TT *)q, (const TT *)k, (const TT *)state, W, U, (TT *)out, (TT *)final_state, (float *)delta, \
        status, T_, nc);                                                                                 \
  } while (0)
  if (dtype == T2FW_F16) T2FW_LAUNCH(__half); else T2FW_LAUNCH(__nv_bfloat16);
#undef T2FW_LAUNCH
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw

#ifdef T2FW_DFW_PROFILE
extern "C" int t2fw_debug_dfw_prof(long long *out) {
  return (int)cudaMemcpyFromSymbol(out, t2fw::g_dfw_prof, sizeof(long long) * 16);
}
#endif
