// Self-test of the tcgen05 primitives in umma.cuh: two M = 64 products computed by the tensor
// core into the two interleaved lane sets of tensor memory and read back with tcgen05.ld.
//
//   D1[64 x N] = A1[64 x Kc] * B1[N x Kc]^T     (tensor-memory lane offset 0)
//   D2[64 x N] = A2[64 x Kc] * B2[N x Kc]^T     (tensor-memory lane offset 16)
//
// The operands arrive as plain row-major fp32 arrays in global memory and are written into
// shared memory either as K-major or as MN-major core-matrix tiles, so that all four operand
// orientations of the production kernels can be checked against a host matrix product.
#include "common.cuh"
#include "lfw_c64.cuh"
#include "umma.cuh"

namespace t2fw {

using namespace umma;

namespace {

constexpr int kM = 64;

__global__ void __launch_bounds__(128)
umma_selftest_kernel(const float *__restrict__ A1, const float *__restrict__ B1,
                     const float *__restrict__ A2, const float *__restrict__ B2,
                     float *__restrict__ D1, float *__restrict__ D2, int N, int Kc, int a_mn,
                     int b_mn, int *__restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail;

  // tile shapes: K-major tiles are [rows = M/N index][cols = Kc]; MN-major are [rows = Kc][cols = M/N]
  const int a_rows = a_mn ? Kc : kM, a_cols = a_mn ? kM : Kc;
  const int b_rows = b_mn ? Kc : N, b_cols = b_mn ? N : Kc;
  const int a_bytes = tile_bytes(a_rows, a_cols), b_bytes = tile_bytes(b_rows, b_cols);
  unsigned char *tA1 = smem, *tA2 = tA1 + a_bytes, *tB1 = tA2 + a_bytes, *tB2 = tB1 + b_bytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 64);
  // operands -> shared memory tiles
  for (int idx = threadIdx.x; idx < kM * Kc; idx += blockDim.x) {
    const int m = idx / Kc, kk = idx % Kc;
    const int off = a_mn ? tile_off(kk, m, a_cols) : tile_off(m, kk, a_cols);
    *reinterpret_cast<float *>(tA1 + off) = A1[idx];
    *reinterpret_cast<float *>(tA2 + off) = A2[idx];
  }
  for (int idx = threadIdx.x; idx < N * Kc; idx += blockDim.x) {
    const int n = idx / Kc, kk = idx % Kc;
    const int off = b_mn ? tile_off(kk, n, b_cols) : tile_off(n, kk, b_cols);
    *reinterpret_cast<float *>(tB1 + off) = B1[idx];
    *reinterpret_cast<float *>(tB2 + off) = B2[idx];
  }
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tbase = tmem_slot;

  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_tf32(kM, N, a_mn != 0, b_mn != 0);
    for (int pair = 0; pair < 2; ++pair) {
      const uint32_t ta = smem_u32(pair ? tA2 : tA1), tb = smem_u32(pair ? tB2 : tB1);
      const uint32_t d = tmem_addr(tbase, pair * 16, 0);
      for (int ks = 0; ks < Kc / 8; ++ks) {
        const uint64_t da = a_mn ? desc_mnmajor(ta, a_cols, 0, ks) : desc_kmajor(ta, a_cols, 0, ks);
        const uint64_t db = b_mn ? desc_mnmajor(tb, b_cols, 0, ks) : desc_kmajor(tb, b_cols, 0, ks);
        mma_tf32(d, da, db, idesc, ks > 0);
      }
    }
    mma_commit(&bar);
  }
  if (!mbar_wait(&bar, 0)) s_fail = 1;
  __syncthreads();
  fence_after_sync();
  if (!s_fail) {
    // warp w reads lanes 32w..32w+31: lanes 0-15 hold rows 16w.. of D1, lanes 16-31 rows of D2
    const int row = 16 * warp + (lane & 15);
    float *dst = (lane < 16 ? D1 : D2) + (size_t)row * N;
    for (int c0 = 0; c0 < N; c0 += 16) {
      float v[16];
      tmem_ld16(tmem_addr(tbase, 32 * warp, c0), v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (c0 + j < N) dst[c0 + j] = v[j];
    }
  } else if (threadIdx.x == 0) {
    atomicExch(status, 1);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 64);
}

// bf16 variant: operands arrive as fp32, are rounded to bf16 in the kernel; both orientations
__global__ void __launch_bounds__(128)
umma_selftest16_kernel(const float *__restrict__ A1, const float *__restrict__ B1,
                       const float *__restrict__ A2, const float *__restrict__ B2,
                       float *__restrict__ D1, float *__restrict__ D2, int N, int Kc, int a_mn,
                       int b_mn, int *__restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail;
  const int a_rows = a_mn ? Kc : kM, a_cols = a_mn ? kM : Kc;
  const int b_rows = b_mn ? Kc : N, b_cols = b_mn ? N : Kc;
  const int a_bytes = tile16_bytes(a_rows, a_cols), b_bytes = tile16_bytes(b_rows, b_cols);
  unsigned char *tA1 = smem, *tA2 = tA1 + a_bytes, *tB1 = tA2 + a_bytes, *tB2 = tB1 + b_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 64);
  for (int idx = threadIdx.x; idx < kM * Kc; idx += blockDim.x) {
    const int m = idx / Kc, kk = idx % Kc;
    const int off = a_mn ? tile16_off(kk, m, a_cols) : tile16_off(m, kk, a_cols);
    *reinterpret_cast<__nv_bfloat16 *>(tA1 + off) = __float2bfloat16_rn(A1[idx]);
    *reinterpret_cast<__nv_bfloat16 *>(tA2 + off) = __float2bfloat16_rn(A2[idx]);
  }
  for (int idx = threadIdx.x; idx < N * Kc; idx += blockDim.x) {
    const int n = idx / Kc, kk = idx % Kc;
    const int off = b_mn ? tile16_off(kk, n, b_cols) : tile16_off(n, kk, b_cols);
    *reinterpret_cast<__nv_bfloat16 *>(tB1 + off) = __float2bfloat16_rn(B1[idx]);
    *reinterpret_cast<__nv_bfloat16 *>(tB2 + off) = __float2bfloat16_rn(B2[idx]);
  }
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tbase = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_16(kM, N, a_mn != 0, b_mn != 0, 1);
    for (int pair = 0; pair < 2; ++pair) {
      const uint32_t ta = smem_u32(pair ? tA2 : tA1), tb = smem_u32(pair ? tB2 : tB1);
      const uint32_t d = tmem_addr(tbase, pair * 16, 0);
      for (int ks = 0; ks < Kc / 16; ++ks) {
        const uint64_t da = a_mn ? desc16_mnmajor(ta, a_cols, 0, ks) : desc16_kmajor(ta, a_cols, 0, ks);
        const uint64_t db = b_mn ? desc16_mnmajor(tb, b_cols, 0, ks) : desc16_kmajor(tb, b_cols, 0, ks);
        mma_f16(d, da, db, idesc, ks > 0);
      }
    }
    mma_commit(&bar);
  }
  if (!mbar_wait(&bar, 0)) s_fail = 1;
  __syncthreads();
  fence_after_sync();
  if (!s_fail) {
    const int row = 16 * warp + (lane & 15);
    float *dst = (lane < 16 ? D1 : D2) + (size_t)row * N;
    for (int c0 = 0; c0 < N; c0 += 16) {
      float v[16];
      tmem_ld16(tmem_addr(tbase, 32 * warp, c0), v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (c0 + j < N) dst[c0 + j] = v[j];
    }
  } else if (threadIdx.x == 0) {
    atomicExch(status, 1);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 64);
}

// A operand from tensor memory: D[64 x 64] = A[64 x 64] * B[64 x 64]^T with A written into tensor
// memory by tcgen05.st and B a 128-byte-swizzle tile in shared memory.  The tensor core reads row r
// of A from the lane in which it produces row r of D, so A and D of one instruction share a lane
// set: A is stored twice (lanes 0-15 and lanes 16-31 of every lane quarter) and each lane set
// computes one 32-column half of D.
__global__ void __launch_bounds__(128)
umma_ts_selftest_kernel(const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ D,
                        int *__restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *tB = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail;
  const int warp = c64::uniform_warp_idx(), lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 2);
    mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) tmem_alloc(&tmem_slot, 128);
  for (int idx = threadIdx.x; idx < 64 * 64; idx += blockDim.x)
    *reinterpret_cast<float *>(tB + c64::toff(idx / 64, idx % 64)) = B[idx];
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tbase = __shfl_sync(0xffffffffu, tmem_slot, 0);
  constexpr int cA = 32, cD = 0;
  {   // A -> tensor memory: both lane sets of this warp's lane quarter hold rows 16 * warp .. + 15
    const int row = 16 * warp + (lane & 15);
    for (int c0 = 0; c0 < 64; c0 += 16) {
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = A[row * 64 + c0 + j];
      tmem_st16(tmem_addr(tbase, 32 * warp, cA + c0), v);
    }
    tmem_st_wait();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  if (warp < 2) {      // one issuing lane per 32-column half
    const uint64_t db = c64::desc_sw128(smem_u32(tB)) + (uint64_t)(warp * 32 * 128 >> 4);
    constexpr uint32_t idesc = make_idesc_tf32(64, 32, false, false);
    const uint32_t d = tmem_addr(tbase, 16 * warp, cD), a0 = tmem_addr(tbase, 16 * warp, cA);
    if (c64::elect_one()) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t o = (uint64_t)(((ks >> 2) * c64::kColBlock + (ks & 3) * 32) >> 4);
        c64::mma_tf32_ts(d, a0 + 8 * ks, db + o, idesc, ks > 0);
      }
      mma_commit(&bar);
    }
    __syncwarp();
  }
  if (!mbar_wait(&bar, 0)) s_fail = 1;
  __syncthreads();
  fence_after_sync();
  if (!s_fail) {
    // every lane executes the warp-collective load; lanes 0-15 hold columns 0-31, lanes 16-31 columns 32-63
    const int row = 16 * warp + (lane & 15), half = lane >> 4;
    for (int c0 = 0; c0 < 32; c0 += 16) {
      float v[16];
      tmem_ld16(tmem_addr(tbase, 32 * warp, cD + c0), v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) D[row * 64 + 32 * half + c0 + j] = v[j];
    }
  } else if (threadIdx.x == 0) {
    atomicExch(status, 1);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 128);
}

}  // namespace

}  // namespace t2fw

using namespace t2fw;

namespace t2fw {
int lfw_chunk_status_ptr(int **out);   // lfw_c64_local.cu
namespace {
// A wait that cannot complete: the barrier expects one arrival and nothing ever arrives.  Nothing
// else is in flight, so giving up is harmless; the kernel reports it exactly as the production
// kernels do (through the status word) and returns.
__global__ void bounded_wait_selftest_kernel(uint32_t limit, int *status) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (!mbar_wait(&bar, 0, limit) && threadIdx.x == 0) atomicExch(status, 1);
}
}  // namespace
}  // namespace t2fw

extern "C" int t2fw_selftest_bounded_wait(int polls, int *status, void *stream) {
  T2FW_CHECK_ARG(polls >= 1 && polls <= 4096, "selftest_bounded_wait: polls in [1, 4096]");
  if (status == nullptr) {      // report through the library's own status word (t2fw_device_status)
    const int rc = lfw_chunk_status_ptr(&status);
    if (rc != T2FW_OK) return rc;
  }
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((uint32_t)polls, status);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

extern "C" int t2fw_selftest_umma_ts(const float *A, const float *B, float *D, int *status, void *stream) {
  T2FW_CHECK_ARG(A && B && D && status, "null pointer argument");
  const int smem = 64 * 64 * 4 + 1024;
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(umma_ts_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  umma_ts_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(A, B, D, status);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

extern "C" int t2fw_selftest_umma16(const float *A1, const float *B1, const float *A2, const float *B2,
                                    float *D1, float *D2, int N, int Kc, int a_mn, int b_mn,
                                    int *status, void *stream) {
  T2FW_CHECK_ARG(A1 && B1 && A2 && B2 && D1 && D2 && status, "null pointer argument");
  T2FW_CHECK_ARG(N >= 8 && N <= 64 && N % 8 == 0 && Kc >= 16 && Kc <= 64 && Kc % 16 == 0,
                 "selftest16: N multiple of 8 in [8, 64], Kc multiple of 16 in [16, 64]");
  const int a_bytes = a_mn ? umma::tile16_bytes(Kc, 64) : umma::tile16_bytes(64, Kc);
  const int b_bytes = b_mn ? umma::tile16_bytes(Kc, N) : umma::tile16_bytes(N, Kc);
  const size_t smem = 2 * (size_t)a_bytes + 2 * (size_t)b_bytes;
  umma_selftest16_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(A1, B1, A2, B2, D1, D2, N,
                                                                             Kc, a_mn, b_mn, status);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

extern "C" int t2fw_selftest_umma(const float *A1, const float *B1, const float *A2, const float *B2,
                                  float *D1, float *D2, int N, int Kc, int a_mn, int b_mn,
                                  int *status, void *stream) {
  T2FW_CHECK_ARG(A1 && B1 && A2 && B2 && D1 && D2 && status, "null pointer argument");
  // The un-swizzled MN-major shared-memory form does not exist for 32-bit operands (the tensor
  // core returns zeros); the production kernels therefore keep every TF32 operand K-major.
  T2FW_CHECK_ARG(a_mn == 0 && b_mn == 0, "selftest: TF32 operands must be K-major (a_mn = b_mn = 0)");
  T2FW_CHECK_ARG(N >= 8 && N <= 64 && N % 8 == 0 && Kc >= 8 && Kc <= 64 && Kc % 8 == 0,
                 "selftest: N and Kc must be multiples of 8 in [8, 64]");
  const int a_bytes = a_mn ? umma::tile_bytes(Kc, 64) : umma::tile_bytes(64, Kc);
  const int b_bytes = b_mn ? umma::tile_bytes(Kc, N) : umma::tile_bytes(N, Kc);
  const size_t smem = 2 * (size_t)a_bytes + 2 * (size_t)b_bytes;
  T2FW_CHECK_CUDA(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
  umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(A1, B1, A2, B2, D1, D2, N, Kc,
                                                                           a_mn, b_mn, status);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}
