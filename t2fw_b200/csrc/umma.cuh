// tcgen05 (5th-generation tensor core) primitives for sm_100a: tensor-memory allocation,
// shared-memory matrix descriptors, MMA issue, completion tracking and accumulator loads.
//
// Operand tiles live in shared memory in the un-swizzled "core matrix" form: 8 x 16-byte
// blocks (8 rows of 4 floats) stored contiguously (128 bytes), row groups and column groups at
// programmable strides.  One physical tile serves both operand orientations:
//   K-major  (tile rows = M/N index, tile columns = contraction index):
//       SBO = stride between 8-row groups, LBO = stride between 4-column groups
//   MN-major (tile rows = contraction index, tile columns = M/N index):
//       SBO = stride between 4-column groups, LBO = stride between 8-row groups
// Accumulators live in tensor memory; an M = 64 tile occupies 16 lanes of each 32-lane quarter,
// so two M = 64 tiles (lane offsets 0 and 16) fill the quarters and a warp's tcgen05.ld sees
// tile 0 in lanes 0-15 and tile 1 in lanes 16-31.
//
// Every wait is bounded: mbar_wait() gives up after a fixed number of polls and returns false.
#pragma once

#include <cstdint>

namespace t2fw {
namespace umma {

// ---- shared-memory tile geometry ---------------------------------------------------------
constexpr int kColGroupBytes = 144;   // 128-byte core matrix + 16 bytes so that 32 consecutive
                                      // columns fall into 32 different banks
// bytes from the tile base to element (r, c) of a tile with `cols` columns (cols % 4 == 0)
__host__ __device__ constexpr int tile_row_group_bytes(int cols) { return (cols / 4) * kColGroupBytes; }
__host__ __device__ constexpr int tile_bytes(int rows, int cols) {
  return ((rows + 7) / 8) * tile_row_group_bytes(cols);
}
__device__ __forceinline__ int tile_off(int r, int c, int cols) {
  return (r & 7) * 16 + (c & 3) * 4 + (r >> 3) * tile_row_group_bytes(cols) + (c >> 2) * kColGroupBytes;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- descriptors ----------------------------------------------------------------------------
// 64-bit shared-memory matrix descriptor, no swizzle, version 1 (sm_100).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
// operand whose tile rows are the M/N index (contraction along tile columns), k-step ks (8 cols)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int cols, int row0, int ks) {
  const uint32_t a = tile_addr + (row0 >> 3) * tile_row_group_bytes(cols) + ks * 2 * kColGroupBytes;
  return make_desc(a, kColGroupBytes, tile_row_group_bytes(cols));
}
// operand whose tile columns are the M/N index (contraction along tile rows), k-step ks (8 rows)
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int cols, int col0, int ks, int row0 = 0) {
  const uint32_t a = tile_addr + ((row0 >> 3) + ks) * tile_row_group_bytes(cols) + (col0 >> 2) * kColGroupBytes;
  return make_desc(a, tile_row_group_bytes(cols), kColGroupBytes);
}
// 32-bit instruction descriptor: TF32 x TF32 -> F32, dense
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N, bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- 16-bit operand tiles (bf16 / fp16): core matrix = 8 rows x 8 elements (16 bytes per row) --
constexpr int kColGroupBytes16 = 144;
__host__ __device__ constexpr int tile16_row_group_bytes(int cols) { return (cols / 8) * kColGroupBytes16; }
__host__ __device__ constexpr int tile16_bytes(int rows, int cols) {
  return ((rows + 7) / 8) * tile16_row_group_bytes(cols);
}
__device__ __forceinline__ int tile16_off(int r, int c, int cols) {
  return (r & 7) * 16 + (c & 7) * 2 + (r >> 3) * tile16_row_group_bytes(cols) + (c >> 3) * kColGroupBytes16;
}
// K-major view (tile rows = M/N index, contraction along tile columns), k-step = 16 columns
__device__ __forceinline__ uint64_t desc16_kmajor(uint32_t tile_addr, int cols, int row0, int ks) {
  const uint32_t a = tile_addr + (row0 >> 3) * tile16_row_group_bytes(cols) + ks * 2 * kColGroupBytes16;
  return make_desc(a, kColGroupBytes16, tile16_row_group_bytes(cols));
}
// MN-major view (tile columns = M/N index, contraction along tile rows), k-step = 16 rows
__device__ __forceinline__ uint64_t desc16_mnmajor(uint32_t tile_addr, int cols, int col0, int ks, int row0 = 0) {
  const uint32_t a = tile_addr + ((row0 >> 3) + 2 * ks) * tile16_row_group_bytes(cols) + (col0 >> 3) * kColGroupBytes16;
  return make_desc(a, tile16_row_group_bytes(cols), kColGroupBytes16);
}
// instruction descriptor: BF16 x BF16 -> F32 (fmt 1) or F16 x F16 -> F32 (fmt 0), dense
__host__ __device__ constexpr uint32_t make_idesc_16(int M, int N, bool a_mn, bool b_mn, int fmt) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((a_mn ? 1u : 0u) << 15) |
         ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------
// One full warp allocates `cols` columns (power of two >= 32); the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col) {
  return base + ((uint32_t)lane << 16) + (uint32_t)col;
}

// ---- MMA, completion -------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]^T, issued by ONE thread.
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
// all MMAs issued so far by this thread arrive on the mbarrier when they complete
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// generic-proxy shared-memory writes -> visible to the tensor core / copy engines
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
constexpr uint32_t kSpinLimit = 1u << 19;
// bounded wait for the phase with the given parity; false on timeout
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 2000;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// ---- accumulator loads: thread i of the warp reads lane (lane field of addr) + i ------------
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t addr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(addr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld4(uint32_t addr, float (&v)[4]) {
  uint32_t r[4];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}
// accumulator stores: thread i of the warp writes lane (lane field of addr) + i, 16 columns
__device__ __forceinline__ void tmem_st16(uint32_t addr, const float *v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(addr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
      "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
      "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
      "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
      "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// barrier among `nthreads` threads (a multiple of 32) that all name the same id (1..15)
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace umma
}  // namespace t2fw
