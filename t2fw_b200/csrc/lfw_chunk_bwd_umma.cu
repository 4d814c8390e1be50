// Main kernel of the chunked decay-rule backward on the tcgen05 tensor core (D = K = 64).
//
// Same mathematics as lfw_chunk_bwd_main.cu (which stays as the mma.sync fallback), organised
// for the Blackwell tensor core:
//   * every operand is kept as a pair of bf16 tiles (hi + lo = 16 mantissa bits) in the
//     un-swizzled core-matrix form, stored [feature][time]; the same tile is read K-major
//     when a product contracts over time and MN-major when it contracts over features, so no
//     transposed copies exist.  A product of two split operands is three MMAs (hi*hi, hi*lo,
//     lo*hi) with fp32 accumulation in tensor memory.
//   * every result is feature-major: a [64 features x 16 steps] accumulator whose rows are
//     tensor-memory lanes, so that after tcgen05.ld a thread holds ONE feature over four steps
//     of a sub-block and the prefix / suffix sums of the gate gradients are register-local up
//     to one exchange between the four warps of a lane quarter.  k-side results live in
//     tensor-memory lanes 0-15 of each quarter, d-side results in lanes 16-31, so the two
//     halves of every warp run the same code on the two sides.
//   * the forward states S[0..3] at the starts of the four sub-blocks are built once per chunk
//     and stay in tensor memory (fp32); the state gradient R stays in registers (fp32).
//   * 16 worker warps (lane quarter x column / step quarter) do the register work; 4 helper
//     warps issue the MMAs (one elected thread each: a thread issues a small MMA only every
//     ~55 cycles, the tensor core retires one every ~25), evaluate the exact tiny-gate formula
//     and write the results out.  The MMAs of a sub-block go into one of two accumulator
//     buffers and run while the workers finish the previous sub-block.
//   * the CTA is persistent; the six raw 8 KB input blocks, the start state and the end-of-chunk
//     state gradient of the next chunk are fetched by bulk asynchronous copies while the
//     current chunk is processed.
//
// Per sub-block I (S0 = S[I], R~ = (aI gI^T) .* R_end, Qt = q*gp, Kt = k/gp, dOt = dO*ap, Xt = x/ap):
//   TQ = S0^T dOt + Kt Z^T      T2 = Qt Z        T7 = R~^T Xt       (rows k;  Z = tril(dOt^T Xt))
//   TO = S0 Qt   + Xt P^T       T4 = dOt P       T8 = R~ Kt         (rows d;  P = tril(Qt^T Kt))
//   dq = gp.*TQ   dk = (T2+T7)./gp   dx = (T4+T8)./ap   R_prev = R~ + dOt Qt^T
//   H  = suffix_t[Qt.*TQ - Kt.*T2] + exclusive_prefix_t[Kt.*T7] + sum_d (R~ .* S0);  d_f_key = H./g
//   (d side the same with the roles exchanged; gates below 2^-10 get the exact formula).
#include <type_traits>

#include "async_copy.cuh"
#include "lfw_chunk.cuh"
#include "umma.cuh"

namespace t2fw {

using namespace chunk;

int lfw_chunk_status_ptr(int **out);   // lfw_chunk_local_umma.cu

#ifdef T2FW_BWD_PROFILE
__device__ long long g_prof[32];
#define PROF(i)                                                    \
  do {                                                             \
    if (threadIdx.x == 0 && blockIdx.x == 0) {                     \
      const long long now_ = clock64();                            \
      g_prof[i] += now_ - tprev;                                   \
      tprev = now_;                                                \
    }                                                              \
  } while (0)
#define PROFH(i)                                                   \
  do {                                                             \
    if (threadIdx.x == 512 && blockIdx.x == 0) {                   \
      const long long now_ = clock64();                            \
      g_prof[16 + i] += now_ - hprev;                              \
      hprev = now_;                                                \
    }                                                              \
  } while (0)
#else
#define PROF(i) do { } while (0)
#define PROFH(i) do { } while (0)
#endif

namespace {

constexpr int kParts = 4;                   // column / step quarters
constexpr int kTW = 128 * kParts;           // worker threads: 4 lane quarters x 4 parts
constexpr int kHelpers = 4;                 // helper warps
constexpr int kTAll = kTW + 32 * kHelpers;
constexpr int kCG = umma::kColGroupBytes16;                // 144
constexpr int kTile = umma::tile16_bytes(kDim, kDim);      // 9216
constexpr int kRGs = umma::tile16_row_group_bytes(kSub);   // 288
constexpr int kTileS = umma::tile16_bytes(kSub, kSub);     // 576
constexpr int kStgLd = 64;      // dense rows: a staging tile leaves as one bulk copy
constexpr int kStgBytes = 5 * kSub * kStgLd * 2;
constexpr int kFixCap = 64;     // tiny-gate entries per sub-block
constexpr float kTinyGate = 9.765625e-4f;   // 2^-10
constexpr int kRawBytes = kC * kDim * 2;
constexpr float kBlockLo = 7.888609e-31f, kBlockHi = 1.267651e+30f;   // 2^-100, 2^100
constexpr float kDivProdHi = 1.329228e+36f;                           // 2^120

// shared-memory map (bytes); the lo tile of every pair directly follows its hi tile
constexpr int oQ = 0, oK = 2 * kTile, oX = 4 * kTile, oO = 6 * kTile, oS = 8 * kTile, oR = 10 * kTile;
constexpr int oP = 12 * kTile;                    // [4 blocks][hi, lo] small tiles
constexpr int oZ = oP + 8 * kTileS;
constexpr int oaI = oZ + 8 * kTileS;
constexpr int ogI = oaI + kNSub * kDim * 4;
constexpr int oXc = ogI + kNSub * kDim * 4;       // [2][kTW] floats: scan totals of the parts
constexpr int oC4 = oXc + 2 * kTW * 4;            // [2 buffers][k side, d side][4][64] floats
constexpr int oFixCode = oC4 + 2 * 2 * 4 * kDim * 4;     // [4][kFixCap] int
constexpr int oFixRg = oFixCode + kNSub * kFixCap * 4;   // [4][kFixCap] float: 1 / gate
constexpr int oFixVal = oFixRg + kNSub * kFixCap * 4;    // [2][kFixCap] float: exact gradients
constexpr int oStg = oFixVal + 2 * kFixCap * 4;   // [2 buffers] 5 tiles [16][kStgLd] 16-bit
constexpr int oRaw = oStg + 2 * kStgBytes;        // x, f, q, k, fk, dO raw blocks
constexpr int kSmem = oRaw + 6 * kRawBytes;
static_assert(kSmem + 256 <= 227 * 1024, "shared memory limit");
static_assert(oRaw % 128 == 0 && oStg % 16 == 0, "alignment of the bulk-copy and staging areas");
// The S0 / R~ tiles are double-buffered by sub-block parity; the second buffer lives in the raw
// input area, which is dead between the operand preparation and the prefetch of the next chunk.
constexpr int oS1 = oRaw, oR1 = oRaw + 2 * kTile;
static_assert(4 * kTile <= 6 * kRawBytes, "second tile buffer fits the raw input area");

// tensor-memory columns.  Lanes A = lanes 0-15 of every quarter, lanes B = lanes 16-31.
constexpr int cS = 0;        // A: S[0..3] at 64*I (1..3 first hold Xt Kt^T of the block before);
                             // B: dOt Qt^T of block I+1 at 64*I
constexpr int cTs = 256;     // result buffer 1
constexpr int cRes0 = 320;   // result buffer 0: +0 TQ|TO, +16 T2|T4, +32 T7|T8
constexpr int cPZ = 384;     // A: P, B: Z (whole chunk)

// named barriers: 1-4 = the four warps of a lane quarter, then
constexpr int kBarH = 5;     // the helper warps among themselves
constexpr int kBarA = 6;     // workers -> helpers: tiles of a block published
constexpr int kBarB = 7;     // (7, 8) workers -> helpers: staging of a block complete
constexpr int kBarY = 9;     // (9, 10) helpers -> workers: exact path done, earlier staging written out

__device__ __forceinline__ void sync_all() {
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
}

__device__ __forceinline__ void split2(float a, float b, uint32_t &hi, uint32_t &lo) {
  const __nv_bfloat162 hh = __floats2bfloat162_rn(a, b);
  const float2 hf = __bfloat1622float2(hh);
  const __nv_bfloat162 ll = __floats2bfloat162_rn(a - hf.x, b - hf.y);
  hi = *reinterpret_cast<const uint32_t *>(&hh);
  lo = *reinterpret_cast<const uint32_t *>(&ll);
}
__device__ __forceinline__ float2 join2(uint32_t hi, uint32_t lo) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&hi));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&lo));
  return make_float2(a.x + b.x, a.y + b.y);
}
// 8 floats -> 8 bf16 (hi) + 8 bf16 (lo) at the same offset of a hi / lo tile pair (lo at +LO)
template <int LO>
__device__ __forceinline__ void write8(unsigned char *th, int off, const float *v) {
  uint4 h, l;
  split2(v[0], v[1], h.x, l.x);
  split2(v[2], v[3], h.y, l.y);
  split2(v[4], v[5], h.z, l.z);
  split2(v[6], v[7], h.w, l.w);
  *reinterpret_cast<uint4 *>(th + off) = h;
  *reinterpret_cast<uint4 *>(th + LO + off) = l;
}
// 4 floats -> 4 + 4 bf16 (8-byte stores)
template <int LO>
__device__ __forceinline__ void write4(unsigned char *th, int off, const float *v) {
  uint2 h, l;
  split2(v[0], v[1], h.x, l.x);
  split2(v[2], v[3], h.y, l.y);
  *reinterpret_cast<uint2 *>(th + off) = h;
  *reinterpret_cast<uint2 *>(th + LO + off) = l;
}
__device__ __forceinline__ void read8(const unsigned char *th, int off, float *v) {
  const uint4 h = *reinterpret_cast<const uint4 *>(th + off);
  const uint4 l = *reinterpret_cast<const uint4 *>(th + kTile + off);
  float2 t;
  t = join2(h.x, l.x); v[0] = t.x; v[1] = t.y;
  t = join2(h.y, l.y); v[2] = t.x; v[3] = t.y;
  t = join2(h.z, l.z); v[4] = t.x; v[5] = t.y;
  t = join2(h.w, l.w); v[6] = t.x; v[7] = t.y;
}
__device__ __forceinline__ void read4(const unsigned char *th, int off, float *v) {
  const uint2 h = *reinterpret_cast<const uint2 *>(th + off);
  const uint2 l = *reinterpret_cast<const uint2 *>(th + kTile + off);
  float2 t;
  t = join2(h.x, l.x); v[0] = t.x; v[1] = t.y;
  t = join2(h.y, l.y); v[2] = t.x; v[3] = t.y;
}
// one element (hi + lo) of a 64-column tile pair
__device__ __forceinline__ float rd1(const unsigned char *th, int r, int c) {
  const int off = umma::tile16_off(r, c, kDim);
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(th + off)) +
         __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(th + kTile + off));
}

// ---- descriptors: low word = start address and leading-dimension offset, high word constant --
// K-major view of a tile with COLS columns: rows = M/N index, 16 columns per k-step.
// MN-major view: columns = M/N index, 16 rows per k-step.
template <bool MN, int COLS>
__device__ __forceinline__ uint32_t dlo(uint32_t tile_addr, int sel, int ks0) {
  constexpr int rg = umma::tile16_row_group_bytes(COLS);
  const uint32_t a = tile_addr + (MN ? 2 * ks0 * rg + (sel >> 3) * kCG : (sel >> 3) * rg + ks0 * 2 * kCG);
  return ((a >> 4) & 0x3FFFu) | ((uint32_t)((MN ? rg : kCG) >> 4) << 16);
}
template <bool MN, int COLS>
__device__ __forceinline__ uint64_t dmake(uint32_t lo, int ks, bool lo_tile) {
  constexpr int rg = umma::tile16_row_group_bytes(COLS);
  constexpr uint32_t hi = (uint32_t)((MN ? kCG : rg) >> 4) | (1u << 14);
  constexpr int pair = (COLS == kDim ? kTile : kTileS) >> 4;
  const uint32_t l = lo + (uint32_t)((MN ? 2 * ks * rg : ks * 2 * kCG) >> 4) + (lo_tile ? pair : 0);
  return ((uint64_t)hi << 32) | l;
}

// D (+)= A * B^T with split operands: hi*hi + hi*lo + lo*hi over NKS k-steps of 16
template <bool AMN, bool BMN, int ACOLS, int BCOLS, int NKS, int N, bool ACC0>
__device__ __forceinline__ void gemm3(uint32_t d, uint32_t a_lo, uint32_t b_lo) {
  constexpr uint32_t idesc = umma::make_idesc_16(kDim, N, AMN, BMN, 1);
#pragma unroll
  for (int ks = 0; ks < NKS; ++ks) {
#pragma unroll
    for (int cmb = 0; cmb < 3; ++cmb)
      umma::mma_f16(d, dmake<AMN, ACOLS>(a_lo, ks, cmb == 2), dmake<BMN, BCOLS>(b_lo, ks, cmb == 1), idesc,
                    ACC0 || ks > 0 || cmb > 0);
  }
}

// producer side of a named barrier: counts this thread without waiting
__device__ __forceinline__ void bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(umma::smem_u32(bar)) : "memory");
}

// sum of a[c] over the 16 lanes of a half warp, for 16 columns c at once: lane fl returns column fl
__device__ __forceinline__ float colsum16(float (&a)[16], int fl) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool up = fl & 8;
    const float send = up ? a[i] : a[i + 8], keep = up ? a[i + 8] : a[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool up = fl & 4;
    const float send = up ? a[i] : a[i + 4], keep = up ? a[i + 4] : a[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool up = fl & 2;
    const float send = up ? a[i] : a[i + 2], keep = up ? a[i + 2] : a[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  const bool up = fl & 1;
  const float send = up ? a[0] : a[1], keep = up ? a[1] : a[0];
  return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

template <typename T>
__global__ void __launch_bounds__(kTAll, 1)
lfw_chunk_bwd_umma_kernel(const T *__restrict__ go, const T *__restrict__ x, const T *__restrict__ f,
                          const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ fk,
                          const T *__restrict__ state, const T *__restrict__ ckpt,
                          const float *__restrict__ Rend, T *__restrict__ dx, T *__restrict__ df,
                          T *__restrict__ dq, T *__restrict__ dk, T *__restrict__ dfk,
                          int *__restrict__ rowflag, int *__restrict__ status, int64_t T_, int64_t nc,
                          int64_t total) {
  extern __shared__ __align__(128) unsigned char sm[];
  __shared__ __align__(8) uint64_t barM[2], barR, barRaw;   // barM: by sub-block parity (pre-phase rounds use [0])
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int s_fail;
  __shared__ int fix_n[kNSub];
  __shared__ unsigned div_max[2];   // largest |divided operand| of the chunk: k side, d side

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool worker = warp < 4 * kParts;
  const int qd = warp & 3, part = (warp >> 2) & 3, side = lane >> 4, fl = lane & 15, feat = 16 * qd + fl;
  const int hw = warp - 4 * kParts;            // helper index 0..3 (helpers only)
  const int ht = threadIdx.x - kTW;            // helper thread 0..127 (helpers only)
  const bool issuer = !worker && lane == 0;

  // per-side views: side 0 = k side (gates fk; Qt, Kt), side 1 = d side (gates f; dOt, Xt)
  unsigned char *mulT = sm + (side ? oO : oQ), *divT = sm + (side ? oX : oK);
  float *blk = reinterpret_cast<float *>(sm + (side ? oaI : ogI));
  const float *aI = reinterpret_cast<const float *>(sm + oaI), *gI = reinterpret_cast<const float *>(sm + ogI);
  float *xc = reinterpret_cast<float *>(sm + oXc);
  float *c4 = reinterpret_cast<float *>(sm + oC4);
  int *fix_code = reinterpret_cast<int *>(sm + oFixCode);
  float *fix_rg = reinterpret_cast<float *>(sm + oFixRg);
  float *fix_val = reinterpret_cast<float *>(sm + oFixVal);
  const T *raw = reinterpret_cast<const T *>(sm + oRaw);   // [6][64][64]: x, f, q, k, fk, dO
  const T *r_gate = raw + (side ? 1 : 4) * kC * kDim;
  const T *r_mul = raw + (side ? 5 : 2) * kC * kDim;
  const T *r_div = raw + (side ? 0 : 3) * kC * kDim;

  auto issue_raw = [&](int64_t ci) {     // thread 0 only
    const int64_t b = ci / nc, c = ci % nc, t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const uint32_t vb = (uint32_t)nv * kDim * sizeof(T);
    const size_t base = ((size_t)b * T_ + t0) * kDim;
    unsigned char *r = sm + oRaw;
    acp::mbar_expect_tx(&barRaw, 6 * vb);
    acp::bulk_g2s(r, x + base, vb, &barRaw);
    acp::bulk_g2s(r + kRawBytes, f + base, vb, &barRaw);
    acp::bulk_g2s(r + 2 * kRawBytes, q + base, vb, &barRaw);
    acp::bulk_g2s(r + 3 * kRawBytes, k + base, vb, &barRaw);
    acp::bulk_g2s(r + 4 * kRawBytes, fk + base, vb, &barRaw);
    acp::bulk_g2s(r + 5 * kRawBytes, go + base, vb, &barRaw);
  };

  bool raw_pending = false;   // thread 0: a prefetch has been issued and not yet awaited
  if (threadIdx.x == 0) {
    umma::mbar_init(&barM[0], kHelpers);
    umma::mbar_init(&barM[1], kHelpers);
    umma::mbar_init(&barR, 1);
    umma::mbar_init(&barRaw, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (threadIdx.x < 2 * kFixCap) fix_val[threadIdx.x] = 0.f;
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 512);
  sync_all();
  const uint32_t tb = tmem_slot;
  const uint32_t tl = umma::tmem_addr(tb, 32 * qd, 0);     // this warp's lane quarter, column 0
  if (threadIdx.x == 0 && (int64_t)blockIdx.x < total) {
    issue_raw(blockIdx.x);
    raw_pending = true;
  }

  const uint32_t aQ = umma::smem_u32(sm + oQ), aK = umma::smem_u32(sm + oK), aX = umma::smem_u32(sm + oX);
  const uint32_t aO = umma::smem_u32(sm + oO), aS0 = umma::smem_u32(sm + oS), aR0 = umma::smem_u32(sm + oR);
  const uint32_t aS1 = umma::smem_u32(sm + oS1), aR1 = umma::smem_u32(sm + oR1);
  const uint32_t aP = umma::smem_u32(sm + oP), aZ = umma::smem_u32(sm + oZ);
  const uint32_t dA = tb, dB = umma::tmem_addr(tb, 16, 0);   // lane sets

  uint32_t pm[2] = {0u, 0u}, pr_ = 0, praw = 0;     // mbarrier phase parities
  // the workers wait for the MMAs of the current round; every helper arrives once per round
  // dOt Qt^T of a block (the first MMAs issued for it): all the next tile publish waits for
  auto wait_rupd = [&]() {
    if (!s_fail && !umma::mbar_wait(&barR, pr_)) s_fail = 1;
    pr_ ^= 1u;
    umma::fence_after_sync();
  };
  // Two barriers, used alternately: the MMAs of a block are committed while the workers may not
  // yet have looked at the barrier of the block before it.
  auto wait_mma = [&](int which) {
    if (!s_fail && !umma::mbar_wait(&barM[which], which ? pm[1] : pm[0])) s_fail = 1;   // after a failure: no more waiting
    if (which) pm[1] ^= 1u; else pm[0] ^= 1u;
    umma::fence_after_sync();
  };

  // Row `feat`, columns 16*part .. +15 of the start-of-chunk state (side 0; 16 packed 16-bit
  // values in the first 8 words) or of the end-of-chunk state gradient (side 1; 16 floats), as
  // raw bits.  Requested one chunk ahead, while R is not live, so the latency is hidden.
  float Rreg[16];   // side 0: S[0] row part (transient); side 1: R~ (persistent over the chunk)
  auto prefetch_rows = [&](int64_t ci) {
    const int64_t b = ci / nc, c = ci % nc;
    if (side == 0) {
      const T *s0 = (c == 0) ? state + (size_t)b * kDim * kDim : ckpt + ((size_t)b * nc + (c - 1)) * kDim * kDim;
      const uint4 *src = reinterpret_cast<const uint4 *>(s0 + feat * kDim + 16 * part);
      const uint4 u0 = src[0], u1 = src[1];
      Rreg[0] = __uint_as_float(u0.x); Rreg[1] = __uint_as_float(u0.y);
      Rreg[2] = __uint_as_float(u0.z); Rreg[3] = __uint_as_float(u0.w);
      Rreg[4] = __uint_as_float(u1.x); Rreg[5] = __uint_as_float(u1.y);
      Rreg[6] = __uint_as_float(u1.z); Rreg[7] = __uint_as_float(u1.w);
    } else {
      const float4 *src = reinterpret_cast<const float4 *>(Rend + (size_t)ci * kDim * kDim + feat * kDim + 16 * part);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 v = src[j];
        Rreg[4 * j] = v.x; Rreg[4 * j + 1] = v.y; Rreg[4 * j + 2] = v.z; Rreg[4 * j + 3] = v.w;
      }
    }
  };
  if (worker && (int64_t)blockIdx.x < total) prefetch_rows(blockIdx.x);

#ifdef T2FW_BWD_PROFILE
  long long tprev = clock64(), hprev = tprev;
#endif
  for (int64_t ci = blockIdx.x; ci < total; ci += gridDim.x) {
    const int64_t b = ci / nc, c = ci % nc, t0c = c * kC;
    const int nvalid = (int)((T_ - t0c < kC) ? T_ - t0c : kC);
    const size_t base = ((size_t)b * T_ + t0c) * kDim;
    PROF(0);
    if (threadIdx.x < kNSub) fix_n[threadIdx.x] = 0;
    if (threadIdx.x < 2) div_max[threadIdx.x] = 0u;
    if (!acp::mbar_wait(&barRaw, praw)) s_fail = 1;
    praw ^= 1u;
    raw_pending = false;
    __syncthreads();
    if (s_fail) break;
    PROF(1);

    // start-of-chunk state (side 0) / end-of-chunk state gradient (side 1): row feat, columns
    // 16*part .. +15
    float pr[kNSub][4], pp0[kNSub];   // this thread's prefix products, kept for the epilogues
    if (worker) {
      if (side == 0) {     // unpack the 16 prefetched 16-bit values, last word first
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          const uint32_t w = __float_as_uint(Rreg[j]);
          const float2 v = Pair<T>::ld(reinterpret_cast<const T *>(&w));
          Rreg[2 * j] = v.x;
          Rreg[2 * j + 1] = v.y;
        }
      }
      // S[0] into tensor memory (lanes A; lanes B receive values that are never read)
      umma::tmem_st16(tl + cS + 16 * part, Rreg);
      PROF(11);

      // ---- operand tiles: thread = (side, feature, step quarter); prefix products restart per block
      bool out_of_range = false;
      float div_hi = 0.f;
#pragma unroll
      for (int I = 0; I < kNSub; ++I) {
        float p = 1.f;
        const int tbk = kSub * I;
#pragma unroll
        for (int j = 0; j < 12; ++j)
          if (j < 4 * part)      // uniform per warp
            p *= sanitize_gate(tbk + j < nvalid ? Elem<T>::ld(r_gate + (tbk + j) * kDim + feat) : 1.f);
        pp0[I] = p;
        const int t0 = tbk + 4 * part;
        float mv[4], dv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int t = t0 + j;
          const bool in = t < nvalid;
          const float pprev = p;
          p *= sanitize_gate(in ? Elem<T>::ld(r_gate + t * kDim + feat) : 1.f);
          pr[I][j] = p;
          mv[j] = (in ? Elem<T>::ld(r_mul + t * kDim + feat) : 0.f) * p;
          dv[j] = __fdividef(in ? Elem<T>::ld(r_div + t * kDim + feat) : 0.f, p);
          if (fabsf(pprev) * kTinyGate > fabsf(p)) {           // |gate| < 2^-10: exact formula later
            const int slot = atomicAdd(&fix_n[I], 1);
            if (slot < kFixCap) {
              fix_code[I * kFixCap + slot] = (side << 16) | ((4 * part + j) << 8) | feat;
              fix_rg[I * kFixCap + slot] = __fdividef(pprev, p);
            } else {
              out_of_range = true;
            }
          }
        }
        // the ratio operands need the sub-block prefix products within [2^-100, 2^100], and the
        // largest divided operand of the k side times that of the d side (they meet in
        // Xt Kt^T) must stay below 2^120: the maxima are collected per side in shared memory
        float plo = fabsf(pr[I][0]), phi = plo, dhi = fabsf(dv[0]);
#pragma unroll
        for (int j = 1; j < 4; ++j) {
          plo = fminf(plo, fabsf(pr[I][j]));
          phi = fmaxf(phi, fabsf(pr[I][j]));
          dhi = fmaxf(dhi, fabsf(dv[j]));
        }
        out_of_range |= !(plo >= kBlockLo && phi <= kBlockHi);
        div_hi = fmaxf(div_hi, dhi);
        const int off = umma::tile16_off(feat, t0, kDim);
        write4<kTile>(mulT, off, mv);
        write4<kTile>(divT, off, dv);
        if (part == kParts - 1) blk[I * kDim + feat] = p;
      }
      PROF(12);
      if (out_of_range) atomicExch(rowflag + b, 1);   // the scan kernels redo this batch row
      {
        const unsigned bits = __float_as_uint(div_hi);     // non-negative floats order like integers
        const unsigned mk = __reduce_max_sync(0xffffffffu, side ? 0u : bits);
        const unsigned md = __reduce_max_sync(0xffffffffu, side ? bits : 0u);
        if (lane == 0) {
          atomicMax(&div_max[0], mk);
          atomicMax(&div_max[1], md);
        }
      }
      umma::tmem_st_wait();
    }
    umma::fence_async_smem();
    sync_all();                       // tiles complete; raw blocks, S0 and R_end buffers consumed
    if (threadIdx.x == 0 && !(__uint_as_float(div_max[0]) * __uint_as_float(div_max[1]) <= kDivProdHi))
      atomicExch(rowflag + b, 1);
    PROF(2);

    // ---- first MMA round: P = Qt^T Kt (lanes A), Z = dOt^T Xt (lanes B) for the whole chunk, and the
    //      local state increments U_J = Xt_J Kt_J^T of blocks 0..2 into the slots of S[1..3] --------
    if (issuer) {
      if (hw == 0) {
        gemm3<true, true, kDim, kDim, 4, kDim, false>(dA + cPZ, dlo<true, kDim>(aQ, 0, 0), dlo<true, kDim>(aK, 0, 0));
      } else if (hw == 1) {
        gemm3<true, true, kDim, kDim, 4, kDim, false>(dB + cPZ, dlo<true, kDim>(aO, 0, 0), dlo<true, kDim>(aX, 0, 0));
      } else if (hw == 2) {
        gemm3<false, false, kDim, kDim, 1, kDim, false>(dA + cS + 64, dlo<false, kDim>(aX, 0, 0), dlo<false, kDim>(aK, 0, 0));
        gemm3<false, false, kDim, kDim, 1, kDim, false>(dA + cS + 128, dlo<false, kDim>(aX, 0, 1), dlo<false, kDim>(aK, 0, 1));
      } else {
        gemm3<false, false, kDim, kDim, 1, kDim, false>(dA + cS + 192, dlo<false, kDim>(aX, 0, 2), dlo<false, kDim>(aK, 0, 2));
      }
      umma::mma_commit(&barM[0]);
    }
    if (worker) wait_mma(0);
    sync_all();
    if (s_fail) break;
    PROF(3);
    if (worker) {
      // diagonal 16 x 16 block of sub-block qd: row fl, columns 4*part .. +3; keep column <= row
      float v[4];
      umma::tmem_ld4(tl + cPZ + 16 * qd + 4 * part, v);
      // forward states at the starts of sub-blocks 1..3 (lanes A), kept in tensor memory:
      // S[J+1] = decay_J .* (S[J] + U_J); lanes B compute on values that are never read
      float u0[16], u1[16], u2[16], sv[16];
      umma::tmem_ld16(tl + cS + 64 + 16 * part, u0);
      umma::tmem_ld16(tl + cS + 128 + 16 * part, u1);
      umma::tmem_ld16(tl + cS + 192 + 16 * part, u2);
      umma::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = (4 * part + j <= fl) ? v[j] : 0.f;
      unsigned char *pt = sm + (side ? oZ : oP) + qd * 2 * kTileS;
      write4<kTileS>(pt, (fl & 7) * 16 + (fl >> 3) * kRGs + (part >> 1) * kCG + (part & 1) * 8, v);
      const float a0 = aI[feat], a1 = aI[kDim + feat], a2 = aI[2 * kDim + feat];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int kc = 16 * part + j;
        sv[j] = (Rreg[j] + u0[j]) * (a0 * gI[kc]);
        u0[j] = sv[j];
        sv[j] = (sv[j] + u1[j]) * (a1 * gI[kDim + kc]);
        u1[j] = sv[j];
        u2[j] = (sv[j] + u2[j]) * (a2 * gI[2 * kDim + kc]);
      }
      umma::tmem_st16(tl + cS + 64 + 16 * part, u0);
      umma::tmem_st16(tl + cS + 128 + 16 * part, u1);
      umma::tmem_st16(tl + cS + 192 + 16 * part, u2);
      umma::tmem_st_wait();
    }
    umma::fence_async_smem();      // the P / Z diagonal blocks written above
    sync_all();
    if (s_fail) break;
    PROF(4);

    // ---- the four sub-blocks in reverse, software-pipelined with producer / consumer barriers:
    //   workers, iteration I: [Y] publish S0 / R~ tiles of block I (A) epilogue of block I+1 (B) wait MMAs(I)
    //   helpers, iteration I: (A) issue MMAs(I), exact path of block I [Y] (B) patch + write-out of block I+1
    //   (A), (B): workers arrive, helpers wait.  [Y]: helpers arrive, workers wait - the tiles of
    //   the previous block are no longer read and the staging buffer of block I+1 has been written out.
#pragma unroll 1
    for (int I = kNSub - 1; I >= -1; --I) {
      const int r0 = kSub * (I < 0 ? 0 : I);
      const int J = I + 1;      // the block whose results are finished in this iteration
      T *stg = reinterpret_cast<T *>(sm + oStg + (J & 1) * kStgBytes);
      if (worker) {
        if (I < 0 && ci + gridDim.x < total) prefetch_rows(ci + gridDim.x);   // R is no longer live
        if (I >= 0 && I < kNSub - 1) wait_rupd();     // dOt Qt^T of block I+1
        if (I >= 0) {
          // lanes A: S[I];  lanes B: dOt Qt^T of block I+1 (the part of R that block added)
          float v[16];
          umma::tmem_ld16(tl + cS + 64 * I + 16 * part, v);
          umma::tmem_ld_wait();
          if (side) {
            const float ar = aI[I * kDim + feat];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float4 g4 = *reinterpret_cast<const float4 *>(gI + I * kDim + 16 * part + 4 * j4);
              const float gg[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int j = 4 * j4 + e;
                const float r = (I == kNSub - 1) ? Rreg[j] : Rreg[j] + v[j];   // R at the end of block I
                Rreg[j] = r * (ar * gg[e]);                                   // R~
                v[j] = Rreg[j];
              }
            }
          }
          unsigned char *th = sm + ((I & 1) ? (side ? oR1 : oS1) : (side ? oR : oS));
          write8<kTile>(th, umma::tile16_off(feat, 16 * part, kDim), v);
          write8<kTile>(th, umma::tile16_off(feat, 16 * part + 8, kDim), v + 8);
          // boundary terms sum_d R~ .* S0 (k side) and sum_k R~ .* S0 (d side): the two half warps
          // exchange their rows (same feature row, same columns), partial sums go to shared memory
          float pd[16], rowsum = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pd[j] = v[j] * __shfl_xor_sync(0xffffffffu, v[j], 16);
            rowsum += pd[j];
          }
          const float colsum = colsum16(pd, fl);
          float *c4b = c4 + (I & 1) * 2 * 4 * kDim;
          if (side) c4b[4 * kDim + part * kDim + feat] = rowsum;       // d side: [part][d]
          else c4b[qd * kDim + 16 * part + fl] = colsum;               // k side: [qd][k]
          umma::fence_async_smem();
          umma::fence_before_sync();
          __threadfence_block();
          bar_arrive(kBarA, kTAll);
        }
        PROF(5);
        if (I < kNSub - 1) {
          wait_mma(J & 1);                                       // every MMA of block J
          umma::named_barrier(kBarY + (J & 1), kTAll);           // the helpers are done with block J's tiles
          umma::fence_after_sync();
          if (I == 0 && threadIdx.x == 0 && ci + gridDim.x < total) {
            issue_raw(ci + gridDim.x);     // block 1 was the last user of the tile buffer in the raw area
            raw_pending = true;
          }
          // ---- feature-major epilogue of block J: this thread = one feature, 4 steps -------------
          const int cres = (J & 1) ? cTs : cRes0;
          float r0v[4], r1v[4], r2v[4];
          umma::tmem_ld4(tl + cres + 4 * part, r0v);
          umma::tmem_ld4(tl + cres + 16 + 4 * part, r1v);
          umma::tmem_ld4(tl + cres + 32 + 4 * part, r2v);
          const float *c4b = c4 + (J & 1) * 2 * 4 * kDim + (side ? 4 * kDim : 0) + feat;
          const float bnd = (c4b[0] + c4b[kDim]) + (c4b[2 * kDim] + c4b[3 * kDim]);
          const int t0 = kSub * J + 4 * part;
          float mr[4], dr[4], p[4];
          const int off = umma::tile16_off(feat, t0, kDim);
          read4(mulT, off, mr);
          read4(divT, off, dr);
#pragma unroll
          for (int j = 0; j < 4; ++j) p[j] = J == 0 ? pr[0][j] : J == 1 ? pr[1][j] : J == 2 ? pr[2][j] : pr[3][j];
          const float pprev0 = J == 0 ? pp0[0] : J == 1 ? pp0[1] : J == 2 ? pp0[2] : pp0[3];
          umma::tmem_ld_wait();
          float o1[4], o2[4], rg[4], V[4], B3[4], pre[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            o1[j] = p[j] * r0v[j];
            rg[j] = __fdividef(1.f, p[j]);
            o2[j] = (r1v[j] + r2v[j]) * rg[j];
            V[j] = mr[j] * r0v[j] - dr[j] * r1v[j];
            B3[j] = dr[j] * r2v[j];
          }
#pragma unroll
          for (int j = 2; j >= 0; --j) V[j] += V[j + 1];          // inclusive suffix over my 4 steps
          float run = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) { pre[j] = run; run += B3[j]; }   // exclusive prefix
          xc[threadIdx.x] = V[0];
          xc[kTW + threadIdx.x] = run;
          umma::named_barrier(1 + qd, 32 * kParts);   // the four warps that share this lane quarter
          float addV = 0.f, addB = 0.f;
#pragma unroll
          for (int pp = 0; pp < kParts; ++pp) {
            const int o = (pp * 4 + qd) * 32 + lane;
            const float tv = xc[o], tbv = xc[kTW + o];
            addV += (pp > part) ? tv : 0.f;          // later steps
            addB += (pp < part) ? tbv : 0.f;         // earlier steps
          }
          T *s1 = stg + (side ? 3 : 1) * kSub * kStgLd, *s2 = stg + (side ? 4 : 2) * kSub * kStgLd;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float H = V[j] + addV + pre[j] + addB + bnd;
            const float pprev = j ? p[j - 1] : pprev0;
            const int lr = 4 * part + j;
            if (!side) stg[lr * kStgLd + feat] = (T)o1[j];
            s1[lr * kStgLd + feat] = (T)o2[j];
            s2[lr * kStgLd + feat] = (T)(H * pprev * rg[j]);
          }
          umma::fence_async_smem();      // the staging tiles are read by the bulk-copy engine
          umma::fence_before_sync();
          __threadfence_block();
          bar_arrive(kBarB + (I & 1), kTAll);
        }
        PROF(6);
      } else {
        if (I >= 0) {
          PROFH(5);
          umma::named_barrier(kBarA, kTAll);
          umma::fence_after_sync();
          PROFH(0);
          if (lane == 0) {
            const int cres = (I & 1) ? cTs : cRes0;
            const uint32_t zI = aZ + I * 2 * kTileS, pI = aP + I * 2 * kTileS;
            const uint32_t aS = (I & 1) ? aS1 : aS0, aR = (I & 1) ? aR1 : aR0;
            if (hw == 0) {
              // dOt Qt^T of this block first, with its own barrier: the tile publish of the next
              // (earlier) sub-block waits for nothing else
              if (I > 0) {
                gemm3<false, false, kDim, kDim, 1, kDim, false>(dB + cS + 64 * (I - 1), dlo<false, kDim>(aO, 0, I),
                                                                dlo<false, kDim>(aQ, 0, I));
                umma::mma_commit(&barR);
              }
              // TQ = S0^T dOt + Kt Z^T
              gemm3<true, true, kDim, kDim, 4, kSub, false>(dA + cres, dlo<true, kDim>(aS, 0, 0), dlo<true, kDim>(aO, r0, 0));
              gemm3<false, false, kDim, kSub, 1, kSub, true>(dA + cres, dlo<false, kDim>(aK, 0, I), dlo<false, kSub>(zI, 0, 0));
            } else if (hw == 1) {
              // T7 = R~^T Xt ;  T2 = Qt Z
              gemm3<true, true, kDim, kDim, 4, kSub, false>(dA + cres + 32, dlo<true, kDim>(aR, 0, 0), dlo<true, kDim>(aX, r0, 0));
              gemm3<false, true, kDim, kSub, 1, kSub, false>(dA + cres + 16, dlo<false, kDim>(aQ, 0, I), dlo<true, kSub>(zI, 0, 0));
            } else if (hw == 2) {
              // TO = S0 Qt + Xt P^T
              gemm3<false, true, kDim, kDim, 4, kSub, false>(dB + cres, dlo<false, kDim>(aS, 0, 0), dlo<true, kDim>(aQ, r0, 0));
              gemm3<false, false, kDim, kSub, 1, kSub, true>(dB + cres, dlo<false, kDim>(aX, 0, I), dlo<false, kSub>(pI, 0, 0));
            } else {
              // T8 = R~ Kt ;  T4 = dOt P
              gemm3<false, true, kDim, kDim, 4, kSub, false>(dB + cres + 32, dlo<false, kDim>(aR, 0, 0), dlo<true, kDim>(aK, r0, 0));
              gemm3<false, true, kDim, kSub, 1, kSub, false>(dB + cres + 16, dlo<false, kDim>(aO, 0, I), dlo<true, kSub>(pI, 0, 0));
            }
            umma::mma_commit(&barM[I & 1]);
          }
          __syncwarp();
          PROFH(1);

          // ---- exact gate gradients of block I where the gate is too small for the cancelling
          //      form (needs only the tiles, so it runs under the MMAs):
          //   dg_t[k] = (1/g_t) sum_d M[d] N[d],  M = S0[d][k] + sum_{i<t} Xt_i[d] Kt_i[k],
          //                                       N = R~[d][k] + sum_{s>=t} dOt_s[d] Qt_s[k]
          // every entry is spread over the four helper warps: 16 values of d per warp, M in the
          // lower half warp and N in the upper one
          const int n_fix = fix_n[I] < kFixCap ? fix_n[I] : kFixCap;
          for (int e = 0; e < n_fix; ++e) {
            const int code = fix_code[I * kFixCap + e];
            const int ds = code >> 16, t = (code >> 8) & 0xff, col = code & 0xff;
            const int o = 16 * hw + (lane & 15), wh = lane >> 4;
            // k-side entry: the fixed feature is a column of S0 / R~, the X / dO rows vary with
            // the lane, the K / Q row of the fixed feature is shared; d side: roles exchanged
            const unsigned char *var = sm + (wh ? (ds ? oQ : oO) : (ds ? oK : oX));
            const unsigned char *fix = sm + (wh ? (ds ? oO : oQ) : (ds ? oX : oK));
            const unsigned char *st0 = sm + ((I & 1) ? (wh ? oR1 : oS1) : (wh ? oR : oS));
            float val = ds ? rd1(st0, col, o) : rd1(st0, o, col);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              float a[8], bb[8];
              read8(var, umma::tile16_off(o, r0 + 8 * h, kDim), a);
              read8(fix, umma::tile16_off(col, r0 + 8 * h, kDim), bb);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const bool use = wh ? (8 * h + i >= t) : (8 * h + i < t);
                val = fmaf(a[i], use ? bb[i] : 0.f, val);
              }
            }
            float mn = val * __shfl_xor_sync(0xffffffffu, val, 16);
#pragma unroll
            for (int sft = 8; sft > 0; sft >>= 1) mn += __shfl_xor_sync(0xffffffffu, mn, sft);
            if (lane == 0) atomicAdd(&fix_val[(I & 1) * kFixCap + e], mn);
          }
          if (ht == 0) acp::bulk_wait_read<0>();   // the earlier write-outs have left shared memory
          __threadfence_block();
          bar_arrive(kBarY + (I & 1), kTAll);
          PROFH(2);
        }
        if (I < kNSub - 1) {
          umma::named_barrier(kBarB + (I & 1), kTAll);
          PROFH(3);
          const int n_fix = fix_n[J] < kFixCap ? fix_n[J] : kFixCap;
          if (ht < n_fix) {
            const int code = fix_code[J * kFixCap + ht];
            const int ds = code >> 16, t = (code >> 8) & 0xff, col = code & 0xff;
            stg[((ds ? 4 : 2) * kSub + t) * kStgLd + col] =
                (T)(fix_val[(J & 1) * kFixCap + ht] * fix_rg[J * kFixCap + ht]);
            fix_val[(J & 1) * kFixCap + ht] = 0.f;      // ready for the next accumulation
          }
          if (n_fix > 0) {
            umma::fence_async_smem();
            umma::named_barrier(kBarH, 32 * kHelpers);
          }
          // ---- the five 16 x 64 result tiles leave as one bulk copy each (rows are contiguous
          //      both in the staging buffer and in the [T][64] output arrays)
          if (ht == 0) {
            const int rJ = kSub * J;
            const int rows = nvalid - rJ < kSub ? nvalid - rJ : kSub;
            if (rows > 0) {
              const uint32_t bytes = (uint32_t)rows * kDim * sizeof(T);
              const size_t o = base + (size_t)rJ * kDim;
              acp::bulk_s2g(dq + o, stg, bytes);
              acp::bulk_s2g(dk + o, stg + kSub * kStgLd, bytes);
              acp::bulk_s2g(dfk + o, stg + 2 * kSub * kStgLd, bytes);
              acp::bulk_s2g(dx + o, stg + 3 * kSub * kStgLd, bytes);
              acp::bulk_s2g(df + o, stg + 4 * kSub * kStgLd, bytes);
            }
            acp::bulk_commit();
          }
          PROFH(4);
        }
      }
    }
    if (ht == 0) acp::bulk_wait_read<0>();   // the last write-out has left the staging buffer
    sync_all();     // nothing of this chunk is in use any more
    if (s_fail) break;
  }
  if (ht == 0) acp::bulk_wait_all();         // every result is in global memory
  if (s_fail && threadIdx.x == 0) {
    atomicExch(status, 1);
    if (raw_pending) acp::mbar_wait(&barRaw, praw);   // bounded: let the copies in flight land
  }
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, 512);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int g_sms[64] = {};

}  // namespace

// returns T2FW_ERR_UNSUPPORTED (without launching) if a pointer is not 16-byte aligned
int lfw_chunk_bwd_main_umma(const void *go, const void *x, const void *f, const void *q, const void *k,
                            const void *fk, const void *state, const void *ckpt, const float *Rend,
                            void *dx, void *df, void *dq, void *dk, void *dfk, int *rowflag, int64_t B,
                            int64_t T_, int dtype, cudaStream_t st) {
  if (!(aligned16(go) && aligned16(x) && aligned16(f) && aligned16(q) && aligned16(k) && aligned16(fk) &&
        aligned16(state) && aligned16(ckpt) && aligned16(Rend) && aligned16(dx) && aligned16(df) &&
        aligned16(dq) && aligned16(dk) && aligned16(dfk)))
    return T2FW_ERR_UNSUPPORTED;
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return T2FW_ERR_UNSUPPORTED;
  if (g_sms[dev] == 0)
    T2FW_CHECK_CUDA(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  const int64_t nc = ceil_div64(T_, kC), total = B * nc;
  const unsigned grid = (unsigned)(total < g_sms[dev] ? total : g_sms[dev]);
#define T2FW_LAUNCH(TT)                                                                               \
  do {                                                                                                \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_chunk_bwd_umma_kernel<TT>,                               \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));        \
    lfw_chunk_bwd_umma_kernel<TT><<<grid, kTAll, kSmem, st>>>(                                        \
        (const TT *)go, (const TT *)x, (const TT *)f, (const TT *)q, (const TT *)k, (const TT *)fk,   \
        (const TT *)state, (const TT *)ckpt, Rend, (TT *)dx, (TT *)df, (TT *)dq, (TT *)dk, (TT *)dfk, \
        rowflag, status, T_, nc, total);                                                              \
  } while (0)
  if (dtype == T2FW_F16) T2FW_LAUNCH(__half); else T2FW_LAUNCH(__nv_bfloat16);
#undef T2FW_LAUNCH
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw

#ifdef T2FW_BWD_PROFILE
extern "C" int t2fw_debug_prof(long long *out) {
  return (int)cudaMemcpyFromSymbol(out, t2fw::g_prof, sizeof(long long) * 32);
}
#endif
