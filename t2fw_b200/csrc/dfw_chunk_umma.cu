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
// processed; Dl and the outputs leave through padded staging rows, copied out with coalesced
// stores while the next products run.  Every wait is bounded.
#include <type_traits>

#include "async_copy.cuh"
#include "lfw_chunk.cuh"
#include "umma.cuh"

namespace t2fw {

using namespace chunk;

int lfw_chunk_status_ptr(int **out);   // lfw_c64_local.cu
int lfw_chunk_sm_count(int *out);


namespace {

constexpr int kTh = 256;                                  // 4 lane quarters x 2 column halves
constexpr int kTileU = umma::tile_bytes(kDim, kC);        // 18432: [64][64] TF32, core-matrix layout
// K and S are adjacent: together they are the 128-row operand of Q [K; S]^T
constexpr int oQ = 0, oW = kTileU, oK = 2 * kTileU, oSt = 3 * kTileU, oAs = 4 * kTileU, oDT = 5 * kTileU,
              oKT = 6 * kTileU;
// K^T is written by transposing scalar stores; with its row groups 16 bytes further apart than
// the dense layout a warp that covers 8 column pieces x 4 steps hits 32 different banks
constexpr int kKTGroup = umma::tile_row_group_bytes(kC) + 16, kKTBytes = (kDim / 8) * kKTGroup;
constexpr int kLdU = kDim + 4;                            // row stride of U tiles in global memory, floats
constexpr int kRow16 = kDim * 2 + 16, kRow32 = kLdU * 4;  // padded staging rows
constexpr int oRawQ = 6 * kTileU + kKTBytes;              // 16-bit [64][64], dense
constexpr int oRawK = oRawQ + kC * kDim * 2;
constexpr int oRawW = oRawK + kC * kDim * 2;              // fp32 [64][64], dense
constexpr int oRawU = oRawW + kC * kDim * 4;              // fp32 [64][kLdU]
constexpr int oStgD = oRawU + kC * kRow32;                // Dl, fp32, row stride kRow32
constexpr int oStgO = oStgD + kC * kRow32;                // outputs, 16-bit, row stride kRow16
constexpr int kSmemU = oStgO + kC * kRow16;
static_assert(kSmemU <= 227 * 1024 && oRawQ % 128 == 0, "shared memory layout");
constexpr int cWS = 0, cSt = 64;                          // tensor-memory columns (both lane sets)
constexpr int kCopyWarp = 7;                              // issues the bulk copies of the next chunk

__device__ __forceinline__ void sync_all() {
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
}
__device__ __forceinline__ int kt_off(int m, int t) {
  return (m & 7) * 16 + (m >> 3) * kKTGroup + (t & 3) * 4 + (t >> 2) * umma::kColGroupBytes;
}
__device__ __forceinline__ uint64_t kt_desc(uint32_t tile_addr, int ks) {
  return umma::make_desc(tile_addr + ks * 2 * umma::kColGroupBytes, umma::kColGroupBytes, kKTGroup);
}
// round to TF32 (nearest, ties away from zero) with one integer addition: the tensor core ignores
// the 13 low mantissa bits.  Infinities and NaNs pass unchanged.
__device__ __forceinline__ float rt(float v) {
  const uint32_t u = __float_as_uint(v);
  return __uint_as_float((u & 0x7f800000u) == 0x7f800000u ? u : u + 0x1000u);
}

template <typename T>
__global__ void __launch_bounds__(kTh, 1)
dfw_chunk_fwd_umma_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ state,
                          const float *__restrict__ W, const float *__restrict__ U, T *__restrict__ out,
                          T *__restrict__ final_state, float *__restrict__ delta, int *__restrict__ status,
                          int64_t T_, int64_t nc) {
  extern __shared__ __align__(128) unsigned char sm[];
  __shared__ __align__(8) uint64_t bar_m1, bar_m2, bar_raw;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;

  const int64_t b = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3, half = warp >> 2, side = lane >> 4, fl = lane & 15;
  const int row = 16 * qd + fl, c0 = 32 * half;
  unsigned char *tS = sm + oSt;

  // one thread: the four raw blocks of a chunk
  auto issue_raw = [&](int64_t c) {
    const int64_t t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const uint32_t vb = (uint32_t)nv * kDim * sizeof(T);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = (size_t)b * nc + c;
    acp::mbar_expect_tx(&bar_raw, 2 * vb + kC * kDim * 4 + kC * kRow32);
    acp::bulk_g2s(sm + oRawW, W + tile * kC * kDim, kC * kDim * 4, &bar_raw);
    acp::bulk_g2s(sm + oRawU, U + tile * kC * kLdU, kC * kRow32, &bar_raw);
    acp::bulk_g2s(sm + oRawQ, q + base, vb, &bar_raw);
    acp::bulk_g2s(sm + oRawK, k + base, vb, &bar_raw);
  };
  // staged outputs of one chunk -> global, 16 bytes per thread and step, consecutive threads
  // consecutive addresses
  auto copy_out_o = [&](int64_t c) {
    const int64_t t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    T *op = out + ((size_t)b * T_ + t0) * kDim;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int p = tid + kTh * j, r = p >> 3, c8 = (p & 7) * 8;
      if (r < nv) *reinterpret_cast<uint4 *>(op + r * kDim + c8) = *reinterpret_cast<const uint4 *>(sm + oStgO + r * kRow16 + c8 * 2);
    }
  };

  if (tid == 0) {
    umma::mbar_init(&bar_m1, 2);
    umma::mbar_init(&bar_m2, 2);
    umma::mbar_init(&bar_raw, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);
  sync_all();
  const uint32_t tb = tmem_slot;
  const uint32_t tl = umma::tmem_addr(tb, 32 * qd, 0);
  if (warp == kCopyWarp && lane == 0) issue_raw(0);

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
        *reinterpret_cast<float4 *>(tS + umma::tile_off(row, c0 + j, kDim)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
    umma::tmem_st16(tl + cSt + c0, v);            // lanes B receive zeros (overwritten by Q S^T)
    umma::tmem_st16(tl + cSt + c0 + 16, v + 16);
    umma::tmem_st_wait();
  }

  uint32_t par = 0;     // all three barriers complete one phase per chunk
  auto wait_bar = [&](uint64_t *bar) {
    if (!s_fail && !umma::mbar_wait(bar, par)) s_fail = 1;
  };

  for (int64_t c = 0; c < nc; ++c) {
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim;
    if (!umma::mbar_wait(&bar_raw, par)) s_fail = 1;    // also after a failure: no copy stays in flight
    __syncthreads();
    if (s_fail) break;

    // ---- raw blocks -> TF32 tiles, in pieces of 4 consecutive columns (1024 per block) -------------
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      {  // Q and W: 16 consecutive lanes cover one row
        const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;
        const uint2 uq = (r < nvalid) ? *reinterpret_cast<const uint2 *>(sm + oRawQ + (r * kDim + c4) * 2) : make_uint2(0u, 0u);
        const float2 q0 = Pair<T>::ld(reinterpret_cast<const T *>(&uq.x)), q1 = Pair<T>::ld(reinterpret_cast<const T *>(&uq.y));
        *reinterpret_cast<float4 *>(sm + oQ + umma::tile_off(r, c4, kDim)) = make_float4(q0.x, q0.y, q1.x, q1.y);
        const float4 w4 = *reinterpret_cast<const float4 *>(sm + oRawW + (r * kDim + c4) * 4);
        *reinterpret_cast<float4 *>(sm + oW + umma::tile_off(r, c4, kDim)) = make_float4(rt(w4.x), rt(w4.y), rt(w4.z), rt(w4.w));
      }
      {  // K and K^T: a warp covers 8 column pieces x 4 steps (see kKTGroup)
        const int combo = warp * 4 + j, r = 4 * (combo >> 1) + (lane >> 3), c4 = 4 * (8 * (combo & 1) + (lane & 7));
        const uint2 uk = (r < nvalid) ? *reinterpret_cast<const uint2 *>(sm + oRawK + (r * kDim + c4) * 2) : make_uint2(0u, 0u);
        const float2 k0 = Pair<T>::ld(reinterpret_cast<const T *>(&uk.x)), k1 = Pair<T>::ld(reinterpret_cast<const T *>(&uk.y));
        *reinterpret_cast<float4 *>(sm + oK + umma::tile_off(r, c4, kDim)) = make_float4(k0.x, k0.y, k1.x, k1.y);
        *reinterpret_cast<float *>(sm + oKT + kt_off(c4, r)) = k0.x;
        *reinterpret_cast<float *>(sm + oKT + kt_off(c4 + 1, r)) = k0.y;
        *reinterpret_cast<float *>(sm + oKT + kt_off(c4 + 2, r)) = k1.x;
        *reinterpret_cast<float *>(sm + oKT + kt_off(c4 + 3, r)) = k1.y;
      }
    }
    // this thread's part of U (lane set A threads): row `row`, columns c0 .. c0+31
    float uv[32];
    if (side == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 u4 = *reinterpret_cast<const float4 *>(sm + oRawU + row * kRow32 + (c0 + j) * 4);
        uv[j] = u4.x; uv[j + 1] = u4.y; uv[j + 2] = u4.z; uv[j + 3] = u4.w;
      }
    }
    if (c > 0) copy_out_o(c - 1);     // staged by the previous chunk, ordered by the barrier above
    umma::fence_async_smem();
    sync_all();                       // tiles complete (the S tile since the end of the last chunk)

    // ---- first round: W S^T (lane set A, columns 0-63) and Q [K; S]^T (lane set B, all columns),
    //      one issuing thread each ---------------------------------------------------------------------
    if (lane == 0 && warp < 2) {
      const uint32_t idesc = umma::make_idesc_tf32(kDim, warp == 0 ? kDim : 2 * kDim, false, false);
      const uint32_t aA = umma::smem_u32(sm + (warp == 0 ? oW : oQ)), aB = umma::smem_u32(sm + (warp == 0 ? oSt : oK));
      const uint32_t d = umma::tmem_addr(tb, warp == 0 ? 0 : 16, cWS);
#pragma unroll
      for (int ks = 0; ks < kC / 8; ++ks)
        umma::mma_tf32(d, umma::desc_kmajor(aA, kDim, 0, ks), umma::desc_kmajor(aB, kDim, 0, ks), idesc, ks > 0);
      umma::mma_commit(&bar_m1);
    }
    if (warp == kCopyWarp && lane == 0 && c + 1 < nc) issue_raw(c + 1);
    wait_bar(&bar_m1);
    umma::fence_after_sync();
    {
      // lane set A: Dl = U - W S^T (row t = `row`, columns d);  lane set B: scores (row t, columns i)
      float v[32];
      umma::tmem_ld16(tl + cWS + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + cWS + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      if (side == 0) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = uv[j] - v[j];
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(sm + oStgD + row * kRow32 + (c0 + j) * 4) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
#pragma unroll
        for (int j = 0; j < 32; ++j)      // Dl^T[d][t]
          *reinterpret_cast<float *>(sm + oDT + umma::tile_off(c0 + j, row, kC)) = rt(v[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j < row) ? rt(v[j]) : 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(sm + oAs + umma::tile_off(row, c0 + j, kC)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    }
    umma::fence_async_smem();
    sync_all();
    // ---- second round: O += A Dl, S += Dl^T K ---------------------------------------------------------
    if (lane == 0 && warp < 2) {
      const uint32_t idesc = umma::make_idesc_tf32(kDim, kDim, false, false);
      const uint32_t aA = umma::smem_u32(sm + (warp == 0 ? oAs : oDT)), aD = umma::smem_u32(sm + oDT),
                     aKT = umma::smem_u32(sm + oKT);
      const uint32_t d = umma::tmem_addr(tb, warp == 0 ? 16 : 0, cSt);
#pragma unroll
      for (int ks = 0; ks < kC / 8; ++ks)
        umma::mma_tf32(d, umma::desc_kmajor(aA, kC, 0, ks), warp == 0 ? umma::desc_kmajor(aD, kC, 0, ks) : kt_desc(aKT, ks),
                       idesc, true);
      umma::mma_commit(&bar_m2);
    }
    // Dl of this chunk -> global while the products run
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;
      if (r < nvalid)
        *reinterpret_cast<float4 *>(delta + base + (size_t)r * kDim + c4) = *reinterpret_cast<const float4 *>(sm + oStgD + r * kRow32 + c4 * 4);
    }
    wait_bar(&bar_m2);
    umma::fence_after_sync();
    {
      // lane set B: O (row t, columns d) -> staging;  lane set A: S (row d, columns m) -> TF32 tile
      float v[32];
      umma::tmem_ld16(tl + cSt + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + cSt + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      if (side) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) Pair<T>::st(reinterpret_cast<T *>(&pk[j]), v[2 * j], v[2 * j + 1]);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4 *>(sm + oStgO + row * kRow16 + c0 * 2 + 16 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
      } else if (c + 1 < nc) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(tS + umma::tile_off(row, c0 + j, kDim)) = make_float4(rt(v[j]), rt(v[j + 1]), rt(v[j + 2]), rt(v[j + 3]));
      } else {
        T *fp = final_state + (size_t)b * kDim * kDim + row * kDim + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 2) Pair<T>::st(fp + j, v[j], v[j + 1]);
      }
    }
    par ^= 1u;
    umma::fence_before_sync();   // accumulator reads are ordered before the next chunk's MMAs
  }
  __syncthreads();
  if (!s_fail && nc > 0) copy_out_o(nc - 1);
  if (s_fail && tid == 0) atomicExch(status, 1);
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, 128);
}

// ---- backward, sequential part ----------------------------------------------------------------------
// Chunks in reverse order; per chunk (S: state walked back, R: state gradient)
//   S0 = S_end - Dl^T K ,  E = Ub + Wb R_end^T (= d_value) ,  R_start = R_end + dO^T Q - E^T K
// and S0^T, R_end^T, E of every chunk go to scratch for the chunk-parallel kernel.  Tensor memory:
//   columns  0-63 :  lane set A: Wb R_end^T        lane set B: S (persistent)
//   columns 64-127:  lane set A: R (persistent)    lane set B: unused
// Tiles with the step index as contraction ([.][t]: -Dl^T, K^T, dO^T, Q^T, -E^T) use the shifted
// row-group stride kKTGroup; Wb and the TF32 copy of R the dense one.
constexpr int oBD = 0, oBK = kKTBytes, oBG = 2 * kKTBytes, oBQ = 3 * kKTBytes, oBE = 4 * kKTBytes,
              oBW = 5 * kKTBytes, oBR = oBW + kTileU;
constexpr int oBRawQ = oBR + kTileU;                      // 16-bit [64][64], dense
constexpr int oBRawK = oBRawQ + kC * kDim * 2;
constexpr int oBRawG = oBRawK + kC * kDim * 2;
constexpr int oBRawD = oBRawG + kC * kDim * 2;            // fp32 [64][64], dense
constexpr int oBRawW = oBRawD + kC * kDim * 4;
constexpr int oBRawU = oBRawW + kC * kDim * 4;            // fp32 [64][kLdU]
constexpr int oBStgE = oBRawU + kC * kRow32;              // E, fp32, row stride kRow32
constexpr int kSmemB = oBStgE + kC * kRow32;
static_assert(kSmemB <= 227 * 1024 && oBRawQ % 128 == 0, "shared memory layout");
constexpr int cE = 0, cR = 64;                            // tensor-memory columns

template <typename T>
__global__ void __launch_bounds__(kTh, 1)
dfw_chunk_bwd_seq_umma_kernel(const T *__restrict__ go, const T *__restrict__ gs, const T *__restrict__ q,
                              const T *__restrict__ k, const float *__restrict__ delta,
                              const T *__restrict__ final_state, const float *__restrict__ Wb,
                              const float *__restrict__ Ub, float *__restrict__ ScT, float *__restrict__ RcT,
                              float *__restrict__ Ec, T *__restrict__ dv, T *__restrict__ ds,
                              int *__restrict__ status, int64_t T_, int64_t nc) {
  extern __shared__ __align__(128) unsigned char sm[];
  __shared__ __align__(8) uint64_t bar_m1, bar_m2, bar_raw;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;

  const int64_t b = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3, half = warp >> 2, side = lane >> 4, fl = lane & 15;
  const int row = 16 * qd + fl, c0 = 32 * half;

  auto issue_raw = [&](int64_t c) {     // one thread
    const int64_t t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const uint32_t vb = (uint32_t)nv * kDim * sizeof(T), vd = (uint32_t)nv * kDim * 4u;
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = (size_t)b * nc + c;
    acp::mbar_expect_tx(&bar_raw, 3 * vb + vd + kC * kDim * 4 + kC * kRow32);
    acp::bulk_g2s(sm + oBRawW, Wb + tile * kC * kDim, kC * kDim * 4, &bar_raw);
    acp::bulk_g2s(sm + oBRawU, Ub + tile * kC * kLdU, kC * kRow32, &bar_raw);
    acp::bulk_g2s(sm + oBRawQ, q + base, vb, &bar_raw);
    acp::bulk_g2s(sm + oBRawK, k + base, vb, &bar_raw);
    acp::bulk_g2s(sm + oBRawG, go + base, vb, &bar_raw);
    acp::bulk_g2s(sm + oBRawD, delta + base, vd, &bar_raw);
  };
  // row `row`, columns c0 .. c0+31 of a [d][m] matrix, transposed into a [m][d] scratch tile
  auto store_t = [&](float *dst, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 32; ++j) dst[(size_t)(c0 + j) * kDim + row] = v[j];
  };
  auto store_r_tile = [&](const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 32; j += 4)
      *reinterpret_cast<float4 *>(sm + oBR + umma::tile_off(row, c0 + j, kDim)) =
          make_float4(rt(v[j]), rt(v[j + 1]), rt(v[j + 2]), rt(v[j + 3]));
  };

  if (tid == 0) {
    umma::mbar_init(&bar_m1, 3);
    umma::mbar_init(&bar_m2, 1);
    umma::mbar_init(&bar_raw, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);
  sync_all();
  const uint32_t tb = tmem_slot;
  const uint32_t tl = umma::tmem_addr(tb, 32 * qd, 0);
  if (warp == kCopyWarp && lane == 0) issue_raw(nc - 1);

  // lane set A threads: the incoming state gradient (= R_end of the last chunk); lane set B threads:
  // the final state.  One store per column range serves both lane sets.
  {
    const T *src = (side == 0 ? gs : final_state) + (size_t)b * kDim * kDim + row * kDim + c0;
    float v[32];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 p = Pair<T>::ld(src + 2 * j);
      v[2 * j] = p.x;
      v[2 * j + 1] = p.y;
    }
    if (side == 0) {
      store_r_tile(v);
      store_t(RcT + ((size_t)b * nc + nc - 1) * kC * kDim, v);
    }
    // R into columns 64.., S into columns 0..: each lane set keeps only its own matrix, the other
    // half of either store lands in accumulator space that the first products overwrite or never read
    umma::tmem_st16(tl + cR + c0, v);
    umma::tmem_st16(tl + cR + c0 + 16, v + 16);
    umma::tmem_st16(tl + cE + c0, v);
    umma::tmem_st16(tl + cE + c0 + 16, v + 16);
    umma::tmem_st_wait();
  }

  uint32_t par = 0;
  auto wait_bar = [&](uint64_t *bar) {
    if (!s_fail && !umma::mbar_wait(bar, par)) s_fail = 1;
  };
  for (int64_t c = nc - 1; c >= 0; --c) {
    const int64_t t0 = c * kC;
    const int nvalid = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const size_t base = ((size_t)b * T_ + t0) * kDim, tile = ((size_t)b * nc + c) * kC * kDim;
    if (!umma::mbar_wait(&bar_raw, par)) s_fail = 1;    // also after a failure: no copy stays in flight
    __syncthreads();
    if (s_fail) break;

    // ---- raw blocks -> TF32 tiles.  A warp covers 8 column pieces x 4 steps per instruction. ---------
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int combo = warp * 4 + j, r = 4 * (combo >> 1) + (lane >> 3), c4 = 4 * (8 * (combo & 1) + (lane & 7));
      const bool in = r < nvalid;
      const uint2 z2 = make_uint2(0u, 0u);
      const uint2 uq = in ? *reinterpret_cast<const uint2 *>(sm + oBRawQ + (r * kDim + c4) * 2) : z2;
      const uint2 uk = in ? *reinterpret_cast<const uint2 *>(sm + oBRawK + (r * kDim + c4) * 2) : z2;
      const uint2 ug = in ? *reinterpret_cast<const uint2 *>(sm + oBRawG + (r * kDim + c4) * 2) : z2;
      const float4 d4 = in ? *reinterpret_cast<const float4 *>(sm + oBRawD + (r * kDim + c4) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 w4 = *reinterpret_cast<const float4 *>(sm + oBRawW + (r * kDim + c4) * 4);
      const float2 q0 = Pair<T>::ld(reinterpret_cast<const T *>(&uq.x)), q1 = Pair<T>::ld(reinterpret_cast<const T *>(&uq.y));
      const float2 k0 = Pair<T>::ld(reinterpret_cast<const T *>(&uk.x)), k1 = Pair<T>::ld(reinterpret_cast<const T *>(&uk.y));
      const float2 g0 = Pair<T>::ld(reinterpret_cast<const T *>(&ug.x)), g1 = Pair<T>::ld(reinterpret_cast<const T *>(&ug.y));
      const int o0 = kt_off(c4, r), o1 = kt_off(c4 + 1, r), o2 = kt_off(c4 + 2, r), o3 = kt_off(c4 + 3, r);
      *reinterpret_cast<float *>(sm + oBQ + o0) = q0.x; *reinterpret_cast<float *>(sm + oBQ + o1) = q0.y;
      *reinterpret_cast<float *>(sm + oBQ + o2) = q1.x; *reinterpret_cast<float *>(sm + oBQ + o3) = q1.y;
      *reinterpret_cast<float *>(sm + oBK + o0) = k0.x; *reinterpret_cast<float *>(sm + oBK + o1) = k0.y;
      *reinterpret_cast<float *>(sm + oBK + o2) = k1.x; *reinterpret_cast<float *>(sm + oBK + o3) = k1.y;
      *reinterpret_cast<float *>(sm + oBG + o0) = g0.x; *reinterpret_cast<float *>(sm + oBG + o1) = g0.y;
      *reinterpret_cast<float *>(sm + oBG + o2) = g1.x; *reinterpret_cast<float *>(sm + oBG + o3) = g1.y;
      *reinterpret_cast<float *>(sm + oBD + o0) = -rt(d4.x); *reinterpret_cast<float *>(sm + oBD + o1) = -rt(d4.y);
      *reinterpret_cast<float *>(sm + oBD + o2) = -rt(d4.z); *reinterpret_cast<float *>(sm + oBD + o3) = -rt(d4.w);
      *reinterpret_cast<float4 *>(sm + oBW + umma::tile_off(r, c4, kDim)) = make_float4(rt(w4.x), rt(w4.y), rt(w4.z), rt(w4.w));
    }
    // this thread's part of Ub (lane set A threads): row `row`, columns c0 .. c0+31
    float uv[32];
    if (side == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 u4 = *reinterpret_cast<const float4 *>(sm + oBRawU + row * kRow32 + (c0 + j) * 4);
        uv[j] = u4.x; uv[j + 1] = u4.y; uv[j + 2] = u4.z; uv[j + 3] = u4.w;
      }
    }
    umma::fence_async_smem();
    sync_all();                       // tiles complete (the R tile since the end of the chunk before)

    // ---- first round, one issuing thread per product -------------------------------------------------
    if (lane == 0 && warp < 3) {
      const uint32_t idesc = umma::make_idesc_tf32(kDim, kDim, false, false);
      if (warp == 0) {          // Wb R_end^T  (rows t, columns d)
        const uint32_t aA = umma::smem_u32(sm + oBW), aB = umma::smem_u32(sm + oBR);
#pragma unroll
        for (int ks = 0; ks < kC / 8; ++ks)
          umma::mma_tf32(umma::tmem_addr(tb, 0, cE), umma::desc_kmajor(aA, kDim, 0, ks),
                         umma::desc_kmajor(aB, kDim, 0, ks), idesc, ks > 0);
      } else {                  // S -= Dl^T K   and   R += dO^T Q
        const uint32_t aA = umma::smem_u32(sm + (warp == 1 ? oBD : oBG)), aB = umma::smem_u32(sm + (warp == 1 ? oBK : oBQ));
        const uint32_t d = warp == 1 ? umma::tmem_addr(tb, 16, cE) : umma::tmem_addr(tb, 0, cR);
#pragma unroll
        for (int ks = 0; ks < kC / 8; ++ks) umma::mma_tf32(d, kt_desc(aA, ks), kt_desc(aB, ks), idesc, true);
      }
      umma::mma_commit(&bar_m1);
    }
    if (warp == kCopyWarp && lane == 0 && c > 0) issue_raw(c - 1);
    wait_bar(&bar_m1);
    umma::fence_after_sync();
    {
      // lane set A: E = Ub + Wb R_end^T (row t = `row`, columns d);  lane set B: S0 (row d, columns m)
      float v[32];
      umma::tmem_ld16(tl + cE + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + cE + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      if (side == 0) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += uv[j];
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(sm + oBStgE + row * kRow32 + (c0 + j) * 4) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
#pragma unroll
        for (int j = 0; j < 32; ++j)      // -E^T[d][t]
          *reinterpret_cast<float *>(sm + oBE + kt_off(c0 + j, row)) = -rt(v[j]);
      } else {
        store_t(ScT + tile, v);
      }
    }
    umma::fence_async_smem();
    sync_all();
    // ---- second round: R -= E^T K ----------------------------------------------------------------------
    if (tid == 0) {
      const uint32_t idesc = umma::make_idesc_tf32(kDim, kDim, false, false);
      const uint32_t aA = umma::smem_u32(sm + oBE), aB = umma::smem_u32(sm + oBK);
#pragma unroll
      for (int ks = 0; ks < kC / 8; ++ks)
        umma::mma_tf32(umma::tmem_addr(tb, 0, cR), kt_desc(aA, ks), kt_desc(aB, ks), idesc, true);
      umma::mma_commit(&bar_m2);
    }
    // E of this chunk -> scratch (all rows) and d_value (valid rows) while the product runs
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;
      const float4 e4 = *reinterpret_cast<const float4 *>(sm + oBStgE + r * kRow32 + c4 * 4);
      *reinterpret_cast<float4 *>(Ec + tile + r * kDim + c4) = e4;
      if (r < nvalid) {
        uint2 pk;
        Pair<T>::st(reinterpret_cast<T *>(&pk.x), e4.x, e4.y);
        Pair<T>::st(reinterpret_cast<T *>(&pk.y), e4.z, e4.w);
        *reinterpret_cast<uint2 *>(dv + base + (size_t)r * kDim + c4) = pk;
      }
    }
    wait_bar(&bar_m2);
    umma::fence_after_sync();
    {
      // R_start (row d, columns m) = R_end of the chunk before, or the state gradient at the start
      float v[32];
      umma::tmem_ld16(tl + cR + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + cR + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      if (side == 0) {
        if (c > 0) {
          store_r_tile(v);
          store_t(RcT + tile - (size_t)kC * kDim, v);
        } else {
          T *dp = ds + (size_t)b * kDim * kDim + row * kDim + c0;
#pragma unroll
          for (int j = 0; j < 32; j += 2) Pair<T>::st(dp + j, v[j], v[j + 1]);
        }
      }
    }
    par ^= 1u;
    umma::fence_before_sync();   // accumulator reads are ordered before the next chunk's MMAs
  }
  if (s_fail && tid == 0) atomicExch(status, 1);
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, 128);
}

// ---- backward, chunk-parallel part -------------------------------------------------------------------
// Persistent CTAs, one per SM, each taking every gridDim-th (batch row, chunk):  with X1 = strict_lower(dO Dl^T), X2 = Dl E^T,
// Y = strict_upper(X2) + its mirror image,
//   d_query = dO S0 + X1 K ,   d_key = Dl R_end + X1^T Q - Y K - E S0 .
// E is stored negated, which makes the third and fourth term of d_key accumulate with a plus sign.
// Tensor memory (M = 64 accumulators, lane sets A / B as above):
//   columns  0-63 :  A: d_key               B: d_query
//   columns 64-127:  A: Dl (-E)^T = -X2     B: dO Dl^T
// First round: dO [S0^T; Dl]^T -> lane set B, Dl [R_end^T; -E]^T -> lane set A (128-column products
// over two adjacent tiles), then (-E) S0 onto d_key.  Second round after the masked tiles are
// written: X1 K onto d_query, X1^T Q and (-Y) K onto d_key.
constexpr int oPS = 0, oPD = kTileU, oPR = 2 * kTileU, oPE = 3 * kTileU, oPG = 4 * kTileU, oPX = 5 * kTileU,
              oPXT = 6 * kTileU, oPY = 7 * kTileU, oPK = 8 * kTileU, oPQ = oPK + kKTBytes;
constexpr int oPStgQ = oPQ + kKTBytes, oPStgK = oPStgQ + kC * kRow16;
constexpr int kSmemP = oPStgK + kC * kRow16;
static_assert(kSmemP <= 227 * 1024, "shared memory layout");

template <typename T>
__global__ void __launch_bounds__(kTh, 1)
dfw_chunk_bwd_par_umma_kernel(const T *__restrict__ go, const T *__restrict__ q, const T *__restrict__ k,
                              const float *__restrict__ delta, const float *__restrict__ ScT,
                              const float *__restrict__ RcT, const float *__restrict__ Ec, T *__restrict__ dq,
                              T *__restrict__ dk, int *__restrict__ status, int64_t T_, int64_t nc,
                              int64_t total) {
  extern __shared__ __align__(128) unsigned char sm[];
  __shared__ __align__(8) uint64_t bar_m1, bar_m2;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qd = warp & 3, half = warp >> 2, side = lane >> 4, fl = lane & 15;
  const int row = 16 * qd + fl, c0 = 32 * half;

  if (tid == 0) {
    umma::mbar_init(&bar_m1, 2);
    umma::mbar_init(&bar_m2, 2);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);

  // The inputs of a chunk travel global -> registers -> TF32 tiles in two steps, so that the loads of
  // the next chunk are in flight during the products and land in the tiles as soon as the products
  // that read them have finished.
  float4 rd[4], re[4], rs[4], rr[4];
  uint2 rg[4], rq[4], rk[4];
  auto chunk_base = [&](int64_t ci) { return ((size_t)(ci / nc) * T_ + (ci % nc) * kC) * kDim; };
  auto chunk_valid = [&](int64_t ci) {
    const int64_t t0 = (ci % nc) * kC;
    return (int)((T_ - t0 < kC) ? T_ - t0 : kC);
  };
  // group A (issued under the first round of products): Dl, E, dO;  group B (under the second): S0^T,
  // R_end^T, q, k.  Two bursts of ~44 KB per SM keep the memory system busy more evenly than one.
  auto load_a = [&](int64_t ci) {
    const size_t base = chunk_base(ci), tile = (size_t)ci * kC * kDim;
    const int nv = chunk_valid(ci);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;       // 16 lanes per row
      const bool in = r < nv;
      rd[j] = in ? *reinterpret_cast<const float4 *>(delta + base + (size_t)r * kDim + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
      rg[j] = in ? *reinterpret_cast<const uint2 *>(go + base + (size_t)r * kDim + c4) : make_uint2(0u, 0u);
      re[j] = *reinterpret_cast<const float4 *>(Ec + tile + r * kDim + c4);
    }
  };
  auto load_b = [&](int64_t ci) {
    const size_t base = chunk_base(ci), tile = (size_t)ci * kC * kDim;
    const int nv = chunk_valid(ci);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;
      rs[j] = *reinterpret_cast<const float4 *>(ScT + tile + r * kDim + c4);
      rr[j] = *reinterpret_cast<const float4 *>(RcT + tile + r * kDim + c4);
      const int combo = warp * 4 + j, rt_ = 4 * (combo >> 1) + (lane >> 3), ct = 4 * (8 * (combo & 1) + (lane & 7));
      const bool in2 = rt_ < nv;                                         // 8 column pieces x 4 steps per warp
      rq[j] = in2 ? *reinterpret_cast<const uint2 *>(q + base + (size_t)rt_ * kDim + ct) : make_uint2(0u, 0u);
      rk[j] = in2 ? *reinterpret_cast<const uint2 *>(k + base + (size_t)rt_ * kDim + ct) : make_uint2(0u, 0u);
    }
  };
  auto store_a = [&]() {          // Dl, -E, dO: read by the first round only
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;
      const int o = umma::tile_off(r, c4, kDim);
      *reinterpret_cast<float4 *>(sm + oPD + o) = make_float4(rt(rd[j].x), rt(rd[j].y), rt(rd[j].z), rt(rd[j].w));
      *reinterpret_cast<float4 *>(sm + oPE + o) = make_float4(-rt(re[j].x), -rt(re[j].y), -rt(re[j].z), -rt(re[j].w));
      const float2 g0 = Pair<T>::ld(reinterpret_cast<const T *>(&rg[j].x)), g1 = Pair<T>::ld(reinterpret_cast<const T *>(&rg[j].y));
      *reinterpret_cast<float4 *>(sm + oPG + o) = make_float4(g0.x, g0.y, g1.x, g1.y);
    }
  };
  auto store_sr = [&]() {         // S0^T, R_end^T: read by the first round only
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = tid + kTh * j, r = p >> 4, c4 = (p & 15) * 4;
      const int o = umma::tile_off(r, c4, kDim);
      *reinterpret_cast<float4 *>(sm + oPS + o) = make_float4(rt(rs[j].x), rt(rs[j].y), rt(rs[j].z), rt(rs[j].w));
      *reinterpret_cast<float4 *>(sm + oPR + o) = make_float4(rt(rr[j].x), rt(rr[j].y), rt(rr[j].z), rt(rr[j].w));
    }
  };
  auto store_trans = [&]() {      // Q^T, K^T: read by the second round only
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int combo = warp * 4 + j, rt_ = 4 * (combo >> 1) + (lane >> 3), ct = 4 * (8 * (combo & 1) + (lane & 7));
      const float2 q0 = Pair<T>::ld(reinterpret_cast<const T *>(&rq[j].x)), q1 = Pair<T>::ld(reinterpret_cast<const T *>(&rq[j].y));
      const float2 k0 = Pair<T>::ld(reinterpret_cast<const T *>(&rk[j].x)), k1 = Pair<T>::ld(reinterpret_cast<const T *>(&rk[j].y));
      const int o0 = kt_off(ct, rt_), o1 = kt_off(ct + 1, rt_), o2 = kt_off(ct + 2, rt_), o3 = kt_off(ct + 3, rt_);
      *reinterpret_cast<float *>(sm + oPQ + o0) = q0.x; *reinterpret_cast<float *>(sm + oPQ + o1) = q0.y;
      *reinterpret_cast<float *>(sm + oPQ + o2) = q1.x; *reinterpret_cast<float *>(sm + oPQ + o3) = q1.y;
      *reinterpret_cast<float *>(sm + oPK + o0) = k0.x; *reinterpret_cast<float *>(sm + oPK + o1) = k0.y;
      *reinterpret_cast<float *>(sm + oPK + o2) = k1.x; *reinterpret_cast<float *>(sm + oPK + o3) = k1.y;
    }
  };
  // staged d_query / d_key rows of a chunk -> global, consecutive threads consecutive addresses
  auto copy_out = [&](int64_t ci) {
    const size_t base = chunk_base(ci);
    const int nv = chunk_valid(ci);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int p = tid + kTh * j, r = p >> 3, c8 = (p & 7) * 8;
      if (r < nv) {
        *reinterpret_cast<uint4 *>(dq + base + (size_t)r * kDim + c8) = *reinterpret_cast<const uint4 *>(sm + oPStgQ + r * kRow16 + c8 * 2);
        *reinterpret_cast<uint4 *>(dk + base + (size_t)r * kDim + c8) = *reinterpret_cast<const uint4 *>(sm + oPStgK + r * kRow16 + c8 * 2);
      }
    }
  };

  int64_t ci = blockIdx.x, prev = -1;
  if (ci < total) {
    load_a(ci);
    load_b(ci);
    store_a();
    store_sr();
    store_trans();
  }
  uint32_t par = 0;
  uint32_t tb = 0, tl = 0;
  for (; ci < total; ci += gridDim.x) {
    umma::fence_async_smem();
    sync_all();                   // tiles complete; staging rows of the chunk before complete
    tb = tmem_slot;
    tl = umma::tmem_addr(tb, 32 * qd, 0);
    if (s_fail) break;
    // ---- first round ---------------------------------------------------------------------------------
    if (lane == 0 && warp < 2) {
      const uint32_t i128 = umma::make_idesc_tf32(kDim, 2 * kDim, false, false), i64 = umma::make_idesc_tf32(kDim, kDim, false, false);
      const uint32_t aA = umma::smem_u32(sm + (warp == 0 ? oPG : oPD)), aB = umma::smem_u32(sm + (warp == 0 ? oPS : oPR));
      const uint32_t d = umma::tmem_addr(tb, warp == 0 ? 16 : 0, 0);
#pragma unroll
      for (int ks = 0; ks < kC / 8; ++ks)
        umma::mma_tf32(d, umma::desc_kmajor(aA, kDim, 0, ks), umma::desc_kmajor(aB, kDim, 0, ks), i128, ks > 0);
      if (warp == 1) {
        const uint32_t aE = umma::smem_u32(sm + oPE), aS = umma::smem_u32(sm + oPS);
#pragma unroll
        for (int ks = 0; ks < kC / 8; ++ks)
          umma::mma_tf32(d, umma::desc_kmajor(aE, kDim, 0, ks), umma::desc_kmajor(aS, kDim, 0, ks), i64, true);
      }
      umma::mma_commit(&bar_m1);
    }
    const int64_t next = ci + gridDim.x;
    const bool has_next = next < total;
    if (has_next) load_a(next);
    if (prev >= 0) copy_out(prev);
    if (!umma::mbar_wait(&bar_m1, par)) s_fail = 1;
    umma::fence_after_sync();
    {
      // lane set B: dO Dl^T (row t, columns i) -> X1 and X1^T;  lane set A: -X2 (row t, columns i) -> -Y
      float v[32];
      umma::tmem_ld16(tl + 64 + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + 64 + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      if (side) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j < row) ? rt(v[j]) : 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4 *>(sm + oPX + umma::tile_off(row, c0 + j, kC)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
#pragma unroll
        for (int j = 0; j < 32; ++j) *reinterpret_cast<float *>(sm + oPXT + umma::tile_off(c0 + j, row, kC)) = v[j];
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          // two independent predicated stores (an if / else-if chain compiles to divergent branches)
          const int i = c0 + j;
          const float y = (i == row) ? 0.f : rt(v[j]);
          if (i >= row) *reinterpret_cast<float *>(sm + oPY + umma::tile_off(row, i, kC)) = y;
          if (i > row) *reinterpret_cast<float *>(sm + oPY + umma::tile_off(i, row, kC)) = y;
        }
      }
    }
    umma::fence_async_smem();
    sync_all();
    // ---- second round --------------------------------------------------------------------------------
    if (lane == 0 && warp < 2) {
      const uint32_t idesc = umma::make_idesc_tf32(kDim, kDim, false, false);
      const uint32_t aK = umma::smem_u32(sm + oPK), aQ = umma::smem_u32(sm + oPQ);
      if (warp == 0) {
        const uint32_t aX = umma::smem_u32(sm + oPX);
#pragma unroll
        for (int ks = 0; ks < kC / 8; ++ks)
          umma::mma_tf32(umma::tmem_addr(tb, 16, 0), umma::desc_kmajor(aX, kC, 0, ks), kt_desc(aK, ks), idesc, true);
      } else {
        const uint32_t aXT = umma::smem_u32(sm + oPXT), aY = umma::smem_u32(sm + oPY);
#pragma unroll
        for (int ks = 0; ks < kC / 8; ++ks)
          umma::mma_tf32(umma::tmem_addr(tb, 0, 0), umma::desc_kmajor(aXT, kC, 0, ks), kt_desc(aQ, ks), idesc, true);
#pragma unroll
        for (int ks = 0; ks < kC / 8; ++ks)
          umma::mma_tf32(umma::tmem_addr(tb, 0, 0), umma::desc_kmajor(aY, kC, 0, ks), kt_desc(aK, ks), idesc, true);
      }
      umma::mma_commit(&bar_m2);
    }
    if (has_next) {                   // the first round has finished with these tiles
      store_a();
      load_b(next);
    }
    if (!s_fail && !umma::mbar_wait(&bar_m2, par)) s_fail = 1;
    umma::fence_after_sync();
    {
      // lane set A: d_key, lane set B: d_query (row t, columns m) -> padded 16-bit staging rows
      float v[32];
      umma::tmem_ld16(tl + c0, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + c0 + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) Pair<T>::st(reinterpret_cast<T *>(&pk[j]), v[2 * j], v[2 * j + 1]);
      unsigned char *stg = sm + (side ? oPStgQ : oPStgK) + row * kRow16 + c0 * 2;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4 *>(stg + 16 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    }
    if (has_next) {                   // both rounds have finished with the tiles
      store_sr();
      store_trans();
    }
    prev = ci;
    par ^= 1u;
    umma::fence_before_sync();
  }
  sync_all();
  if (!s_fail && prev >= 0) copy_out(prev);
  if (s_fail && tid == 0) atomicExch(status, 1);
  if (warp == 0) umma::tmem_dealloc(tmem_slot, 128);
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

// sequential part of the backward; same contract as above
int dfw_chunk_bwd_seq_umma(const void *go, const void *gs, const void *q, const void *k, const void *delta,
                           const void *final_state, const float *Wb, const float *Ub, float *ScT, float *RcT,
                           float *Ec, void *dv, void *ds, int64_t B, int64_t T_, int dtype, cudaStream_t st) {
  if (!(aligned16(go) && aligned16(gs) && aligned16(q) && aligned16(k) && aligned16(delta) &&
        aligned16(final_state) && aligned16(Wb) && aligned16(Ub) && aligned16(ScT) && aligned16(RcT) &&
        aligned16(Ec) && aligned16(dv) && aligned16(ds)))
    return T2FW_ERR_UNSUPPORTED;
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  const int64_t nc = ceil_div64(T_, kC);
#define T2FW_LAUNCH(TT)                                                                                  \
  do {                                                                                                   \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_bwd_seq_umma_kernel<TT>,                              \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemB));          \
    dfw_chunk_bwd_seq_umma_kernel<TT><<<(unsigned)B, kTh, kSmemB, st>>>(                                 \
        (const TT *)go, (const TT *)gs, (const TT *)q, (const TT *)k, (const float *)delta,              \
        (const TT *)final_state, Wb, Ub, ScT, RcT, Ec, (TT *)dv, (TT *)ds, status, T_, nc);              \
  } while (0)
  if (dtype == T2FW_F16) T2FW_LAUNCH(__half); else T2FW_LAUNCH(__nv_bfloat16);
#undef T2FW_LAUNCH
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

// chunk-parallel part of the backward; same contract as above
int dfw_chunk_bwd_par_umma(const void *go, const void *q, const void *k, const void *delta, const float *ScT,
                           const float *RcT, const float *Ec, void *dq, void *dk, int64_t B, int64_t T_, int dtype,
                           cudaStream_t st) {
  if (!(aligned16(go) && aligned16(q) && aligned16(k) && aligned16(delta) && aligned16(ScT) && aligned16(RcT) &&
        aligned16(Ec) && aligned16(dq) && aligned16(dk)))
    return T2FW_ERR_UNSUPPORTED;
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return T2FW_ERR_UNSUPPORTED;
  int n_sm = 0;
  {
    const int rc_sm = lfw_chunk_sm_count(&n_sm);     // cached per device under a lock
    if (rc_sm != T2FW_OK) return rc_sm;
  }
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  const int64_t nc = ceil_div64(T_, kC), total = B * nc;
  const unsigned grid = (unsigned)(total < n_sm ? total : n_sm);     // one persistent CTA per SM
#define T2FW_LAUNCH(TT)                                                                                  \
  do {                                                                                                   \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(dfw_chunk_bwd_par_umma_kernel<TT>,                              \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemP));          \
    dfw_chunk_bwd_par_umma_kernel<TT><<<grid, kTh, kSmemP, st>>>(                                        \
        (const TT *)go, (const TT *)q, (const TT *)k, (const float *)delta, ScT, RcT, Ec, (TT *)dq,      \
        (TT *)dk, status, T_, nc, total);                                                                \
  } while (0)
  if (dtype == T2FW_F16) T2FW_LAUNCH(__half); else T2FW_LAUNCH(__nv_bfloat16);
#undef T2FW_LAUNCH
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw

