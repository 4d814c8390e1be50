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
//     tensor-memory lanes, so that after tcgen05.ld a thread holds ONE feature over the steps of
//     a sub-block and all the prefix / suffix sums of the gate gradients are register-local.
//     k-side results live in tensor-memory lanes 0-15 of each quarter, d-side results in lanes
//     16-31, so the two halves of every warp run the same code on the two sides.
//   * the forward states S[0..3] at the starts of the four sub-blocks are built once per chunk
//     and stay in tensor memory (fp32); the state gradient R stays in registers (fp32).
//   * four more warps do nothing but issue MMAs (one elected thread each: a thread issues a
//     small MMA only every ~90 cycles, the tensor core retires one every ~30).  The MMAs of a
//     sub-block go into one of two accumulator buffers and run while the eight worker warps do
//     the register work of the previous sub-block (epilogue, exact tiny-gate path, write-out).
//   * the CTA is persistent; the six raw 8 KB input blocks, the start state and the end-of-chunk
//     state gradient of the next chunk are fetched by bulk asynchronous copies while the
//     current chunk is processed.
//
// Per sub-block I (S0 = S[I], R~ = (aI gI^T) .* R_end, Qt = q*gp, Kt = k/gp, dOt = dO*ap, Xt = x/ap):
//   TQ = S0^T dOt + Kt Z^T      T2 = Qt Z        T7 = R~^T Xt       (rows k;  Z = tril(dOt^T Xt))
//   TO = S0 Qt   + Xt P^T       T4 = dOt P       T8 = R~ Kt         (rows d;  P = tril(Qt^T Kt))
//   dq = gp.*TQ   dk = (T2+T7)./gp   dx = (T4+T8)./ap   R_prev = R~ + dOt Qt^T
//   H  = suffix_t[Qt.*TQ - Kt.*T2] + exclusive_prefix_t[Kt.*T7] + diag(R~^T S0);  d_f_key = H./g
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
#else
#define PROF(i) do { } while (0)
#endif

namespace {

constexpr int kT = 256;        // worker threads: 8 warps = 4 lane quarters x 2 column / step halves
constexpr int kIssuers = 4;
constexpr int kTAll = kT + 32 * kIssuers;   // + warps 8..11: one elected thread each issues MMAs
constexpr int kCG = umma::kColGroupBytes16;                // 144
constexpr int kRG = umma::tile16_row_group_bytes(kDim);    // 1152
constexpr int kTile = umma::tile16_bytes(kDim, kDim);      // 9216
constexpr int kRGs = umma::tile16_row_group_bytes(kSub);   // 288
constexpr int kTileS = umma::tile16_bytes(kSub, kSub);     // 576
constexpr int kStgLd = 72;      // elements per row of the 16-bit output staging tiles
constexpr int kFixCap = 64;     // tiny-gate entries per sub-block
constexpr float kTinyGate = 9.765625e-4f;   // 2^-10
constexpr int kRawBytes = kC * kDim * 2;
constexpr float kBlockLo = 8.673617e-19f, kBlockHi = 1.152922e+18f;   // 2^-60, 2^60
constexpr float kDivHi = 7.205759e+16f;                               // 2^56

// shared-memory map (bytes); the lo tile of every pair directly follows its hi tile
constexpr int oQ = 0, oK = 2 * kTile, oX = 4 * kTile, oO = 6 * kTile, oS = 8 * kTile, oR = 10 * kTile;
constexpr int oP = 12 * kTile;                    // [4 blocks][hi, lo] small tiles
constexpr int oZ = oP + 8 * kTileS;
constexpr int oaI = oZ + 8 * kTileS;
constexpr int ogI = oaI + kNSub * kDim * 4;
constexpr int oXc = ogI + kNSub * kDim * 4;       // [2][256] floats
constexpr int oFixCode = oXc + 2 * kT * 4;        // [4][kFixCap] int
constexpr int oFixRg = oFixCode + kNSub * kFixCap * 4;   // [4][kFixCap] float: 1 / gate
constexpr int oFixVal = oFixRg + kNSub * kFixCap * 4;    // [2][kFixCap] float: exact gradients
constexpr int oStg = oFixVal + 2 * kFixCap * 4;   // 5 tiles [16][kStgLd] 16-bit
constexpr int oRaw = oStg + 5 * kSub * kStgLd * 2;   // x, f, q, k, fk, dO raw blocks
constexpr int oS0 = oRaw + 6 * kRawBytes;         // start-of-chunk state [64][64] 16-bit
constexpr int oRe = oS0 + kRawBytes;              // end-of-chunk state gradient [64][64] fp32
constexpr int kSmem = oRe + kDim * kDim * 4;
static_assert(kSmem <= 227 * 1024, "shared memory budget");
static_assert(oRaw % 128 == 0 && oStg % 16 == 0, "alignment of the bulk-copy and staging areas");

// tensor-memory columns.  Lanes A = lanes 0-15 of every quarter, lanes B = lanes 16-31.
constexpr int cS = 0;        // A: S[0..3] at 64*I;  B: dOt Qt^T of block I+1 at 64*I
constexpr int cTs = 256;     // A: chain accumulator; afterwards result buffer 1
constexpr int cRes0 = 320;   // result buffer 0: +0 TQ|TO, +16 T2|T4, +32 T7|T8
constexpr int cPZ = 384;     // A: P, B: Z (whole chunk); afterwards boundary buffer 1
constexpr int cDg0 = 448;    // boundary buffer 0: A: R~^T S0, B: S0 R~^T (diagonals used)

__device__ __forceinline__ void sync_all() {
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
}

// 8 floats -> 8 bf16 (hi) + 8 bf16 (lo) at the same offset of a hi / lo tile pair (lo at +LO)
template <int LO>
__device__ __forceinline__ void write8(unsigned char *th, int off, const float *v) {
  uint4 h, l;
  uint32_t *hw = reinterpret_cast<uint32_t *>(&h), *lw = reinterpret_cast<uint32_t *>(&l);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 hh = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    const float2 hf = __bfloat1622float2(hh);
    const __nv_bfloat162 ll = __floats2bfloat162_rn(v[2 * j] - hf.x, v[2 * j + 1] - hf.y);
    hw[j] = *reinterpret_cast<const uint32_t *>(&hh);
    lw[j] = *reinterpret_cast<const uint32_t *>(&ll);
  }
  *reinterpret_cast<uint4 *>(th + off) = h;
  *reinterpret_cast<uint4 *>(th + LO + off) = l;
}
__device__ __forceinline__ void read8(const unsigned char *th, int off, float *v) {
  const uint4 h = *reinterpret_cast<const uint4 *>(th + off);
  const uint4 l = *reinterpret_cast<const uint4 *>(th + kTile + off);
  const __nv_bfloat162 *hp = reinterpret_cast<const __nv_bfloat162 *>(&h);
  const __nv_bfloat162 *lp = reinterpret_cast<const __nv_bfloat162 *>(&l);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = __bfloat1622float2(hp[j]), b = __bfloat1622float2(lp[j]);
    v[2 * j] = a.x + b.x;
    v[2 * j + 1] = a.y + b.y;
  }
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

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(umma::smem_u32(bar)) : "memory");
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
  __shared__ __align__(8) uint64_t barM, barRaw;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail, fix_n[kNSub];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qd = warp & 3, half = warp >> 2, side = lane >> 4, fl = lane & 15, feat = 16 * qd + fl;
  const bool worker = warp < 8, issuer = !worker && lane == 0;
  const int iw = warp - 8;   // issuer index 0..3

  // per-side views: side 0 = k side (gates fk; Qt, Kt), side 1 = d side (gates f; dOt, Xt)
  unsigned char *mulT = sm + (side ? oO : oQ), *divT = sm + (side ? oX : oK);
  float *blk = reinterpret_cast<float *>(sm + (side ? oaI : ogI));
  const float *aI = reinterpret_cast<const float *>(sm + oaI), *gI = reinterpret_cast<const float *>(sm + ogI);
  float *xc = reinterpret_cast<float *>(sm + oXc);
  int *fix_code = reinterpret_cast<int *>(sm + oFixCode);
  float *fix_rg = reinterpret_cast<float *>(sm + oFixRg);
  float *fix_val = reinterpret_cast<float *>(sm + oFixVal);
  T *stg = reinterpret_cast<T *>(sm + oStg);
  const T *raw = reinterpret_cast<const T *>(sm + oRaw);   // [6][64][64]: x, f, q, k, fk, dO
  const T *r_gate = raw + (side ? 1 : 4) * kC * kDim;
  const T *r_mul = raw + (side ? 5 : 2) * kC * kDim;
  const T *r_div = raw + (side ? 0 : 3) * kC * kDim;

  auto issue_raw = [&](int64_t ci) {     // thread 0 only
    const int64_t b = ci / nc, c = ci % nc, t0 = c * kC;
    const int nv = (int)((T_ - t0 < kC) ? T_ - t0 : kC);
    const uint32_t vb = (uint32_t)nv * kDim * sizeof(T);
    const size_t base = ((size_t)b * T_ + t0) * kDim;
    const T *s0 = (c == 0) ? state + (size_t)b * kDim * kDim : ckpt + ((size_t)b * nc + (c - 1)) * kDim * kDim;
    unsigned char *r = sm + oRaw;
    acp::mbar_expect_tx(&barRaw, 6 * vb + kRawBytes + kDim * kDim * 4);
    acp::bulk_g2s(r, x + base, vb, &barRaw);
    acp::bulk_g2s(r + kRawBytes, f + base, vb, &barRaw);
    acp::bulk_g2s(r + 2 * kRawBytes, q + base, vb, &barRaw);
    acp::bulk_g2s(r + 3 * kRawBytes, k + base, vb, &barRaw);
    acp::bulk_g2s(r + 4 * kRawBytes, fk + base, vb, &barRaw);
    acp::bulk_g2s(r + 5 * kRawBytes, go + base, vb, &barRaw);
    acp::bulk_g2s(sm + oS0, s0, kRawBytes, &barRaw);
    acp::bulk_g2s(sm + oRe, Rend + (size_t)ci * kDim * kDim, kDim * kDim * 4, &barRaw);
  };

  bool raw_pending = false;   // thread 0: a prefetch has been issued and not yet awaited
  if (threadIdx.x == 0) {
    umma::mbar_init(&barM, kIssuers);
    umma::mbar_init(&barRaw, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 512);
  sync_all();
  const uint32_t tb = tmem_slot;
  const uint32_t tl = umma::tmem_addr(tb, 32 * qd, 0);     // this warp's lane quarter, column 0
  if (threadIdx.x == 0 && (int64_t)blockIdx.x < total) {
    issue_raw(blockIdx.x);
    raw_pending = true;
  }

  const uint32_t aQ = umma::smem_u32(sm + oQ), aK = umma::smem_u32(sm + oK), aX = umma::smem_u32(sm + oX);
  const uint32_t aO = umma::smem_u32(sm + oO), aS = umma::smem_u32(sm + oS), aR = umma::smem_u32(sm + oR);
  const uint32_t aP = umma::smem_u32(sm + oP), aZ = umma::smem_u32(sm + oZ);
  const uint32_t dA = tb, dB = umma::tmem_addr(tb, 16, 0);   // lane sets

  uint32_t pm = 0, praw = 0;     // mbarrier phase parities
  // every thread waits for the MMAs of the current round; all issuers arrive once per round
  auto wait_mma = [&]() {
    if (!umma::mbar_wait(&barM, pm)) s_fail = 1;
    pm ^= 1u;
    umma::fence_after_sync();
  };

#ifdef T2FW_BWD_PROFILE
  long long tprev = clock64();
#endif
  for (int64_t ci = blockIdx.x; ci < total; ci += gridDim.x) {
    const int64_t b = ci / nc, c = ci % nc, t0c = c * kC;
    const int nvalid = (int)((T_ - t0c < kC) ? T_ - t0c : kC);
    const size_t base = ((size_t)b * T_ + t0c) * kDim;
    PROF(0);
    if (threadIdx.x < kNSub) fix_n[threadIdx.x] = 0;
    if (!acp::mbar_wait(&barRaw, praw)) s_fail = 1;
    praw ^= 1u;
    raw_pending = false;
    __syncthreads();
    if (s_fail) break;
    PROF(1);

    // start-of-chunk state (side 0) / end-of-chunk state gradient (side 1): row feat, columns
    // 32*half .. +31
    float Rreg[32];   // side 0: S[0] row half (transient); side 1: R~ (persistent over the chunk)
    float pr[kNSub][8], pp0[kNSub];   // this thread's prefix products, kept for the epilogues
    if (worker) {
    if (side == 0) {
      const T *Sc = reinterpret_cast<const T *>(sm + oS0) + feat * kDim + 32 * half;
#pragma unroll
      for (int j4 = 0; j4 < 4; ++j4) {
        const uint4 u = *reinterpret_cast<const uint4 *>(Sc + 8 * j4);
        const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
        for (int j = 0; j < 8; ++j) Rreg[8 * j4 + j] = Elem<T>::ld(e + j);
      }
    } else {
      const float *Rc = reinterpret_cast<const float *>(sm + oRe) + feat * kDim + 32 * half;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 v = *reinterpret_cast<const float4 *>(Rc + 4 * j);
        Rreg[4 * j] = v.x; Rreg[4 * j + 1] = v.y; Rreg[4 * j + 2] = v.z; Rreg[4 * j + 3] = v.w;
      }
    }
    // S[0] into tensor memory (lanes A; lanes B receive values that are never read)
    umma::tmem_st16(tl + cS + 32 * half, Rreg);
    umma::tmem_st16(tl + cS + 32 * half + 16, Rreg + 16);
    umma::tmem_st16(tl + cTs + 32 * half, Rreg);
    umma::tmem_st16(tl + cTs + 32 * half + 16, Rreg + 16);

    PROF(11);
    // ---- operand tiles: thread = (side, feature, token half); prefix products restart per block
    bool out_of_range = false;
#pragma unroll
    for (int I = 0; I < kNSub; ++I) {
      float p = 1.f;
      const int tbk = kSub * I;
      if (half) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          p *= sanitize_gate(tbk + j < nvalid ? Elem<T>::ld(r_gate + (tbk + j) * kDim + feat) : 1.f);
      }
      pp0[I] = p;
      const int t0 = tbk + 8 * half;
      float mv[8], dv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
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
            fix_code[I * kFixCap + slot] = (side << 16) | ((8 * half + j) << 8) | feat;
            fix_rg[I * kFixCap + slot] = __fdividef(pprev, p);
          } else {
            out_of_range = true;
          }
        }
      }
      // the ratio operands need the sub-block prefix products within [2^-60, 2^60] and the
      // divided operands below 2^56, so that no product of two of them overflows
      float plo = fabsf(pr[I][0]), phi = plo, dhi = fabsf(dv[0]);
#pragma unroll
      for (int j = 1; j < 8; ++j) {
        plo = fminf(plo, fabsf(pr[I][j]));
        phi = fmaxf(phi, fabsf(pr[I][j]));
        dhi = fmaxf(dhi, fabsf(dv[j]));
      }
      out_of_range |= !(plo >= kBlockLo && phi <= kBlockHi && dhi <= kDivHi);
      const int off = umma::tile16_off(feat, t0, kDim);
      write8<kTile>(mulT, off, mv);
      write8<kTile>(divT, off, dv);
      if (half) blk[I * kDim + feat] = p;
    }
    PROF(12);
    if (out_of_range) atomicExch(rowflag + b, 1);   // the scan kernels redo this batch row
    umma::tmem_st_wait();
    }
    umma::fence_async_smem();
    sync_all();                       // tiles complete; raw blocks, S0 and R_end buffers consumed
    if (threadIdx.x == 0 && ci + gridDim.x < total) {
      issue_raw(ci + gridDim.x);
      raw_pending = true;
    }
    PROF(2);

    // ---- round 1: P = Qt^T Kt (lanes A), Z = dOt^T Xt (lanes B) for the whole chunk, and the
    //      first link of the state chain: accumulator (= S[0]) += Xt_0 Kt_0^T ------------------
    if (issuer) {
      if (iw == 0) {
        gemm3<false, false, kDim, kDim, 1, kDim, true>(dA + cTs, dlo<false, kDim>(aX, 0, 0), dlo<false, kDim>(aK, 0, 0));
        gemm3<true, true, kDim, kDim, 4, kDim, false>(dA + cPZ, dlo<true, kDim>(aQ, 0, 0), dlo<true, kDim>(aK, 0, 0));
        umma::mma_commit(&barM);
      } else if (iw == 1) {
        gemm3<true, true, kDim, kDim, 4, kDim, false>(dB + cPZ, dlo<true, kDim>(aO, 0, 0), dlo<true, kDim>(aX, 0, 0));
        umma::mma_commit(&barM);
      } else {
        mbar_arrive(&barM);
      }
    }
    wait_mma();
    sync_all();
    if (s_fail) break;
    PROF(3);
    if (worker) {
      // diagonal 16 x 16 block of sub-block qd: row fl, columns 8*half .. +7; keep column <= row
      float v[8];
      umma::tmem_ld8(tl + cPZ + 16 * qd + 8 * half, v);
      umma::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (8 * half + j <= fl) ? v[j] : 0.f;
      unsigned char *pt = sm + (side ? oZ : oP) + qd * 2 * kTileS;
      write8<kTileS>(pt, (fl & 7) * 16 + (fl >> 3) * kRGs + half * kCG, v);
    }

    // ---- forward states at the starts of sub-blocks 1..3 (lanes A), kept in tensor memory -----
#pragma unroll 1
    for (int J = 0; J + 1 < kNSub; ++J) {
      if (J > 0) {
        if (issuer) {
          // chain accumulator += Xt_J Kt_J^T  (contraction over the 16 steps of block J)
          if (iw == 0) {
            gemm3<false, false, kDim, kDim, 1, kDim, true>(dA + cTs, dlo<false, kDim>(aX, 0, J),
                                                           dlo<false, kDim>(aK, 0, J));
            umma::mma_commit(&barM);
          } else {
            mbar_arrive(&barM);
          }
        }
        wait_mma();
        sync_all();
        if (s_fail) break;
      }
      if (worker) {
      float v[32];
      umma::tmem_ld16(tl + cTs + 32 * half, *reinterpret_cast<float(*)[16]>(v));
      umma::tmem_ld16(tl + cTs + 32 * half + 16, *reinterpret_cast<float(*)[16]>(v + 16));
      umma::tmem_ld_wait();
      const float ar = aI[J * kDim + feat];
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        const float4 g4 = *reinterpret_cast<const float4 *>(gI + J * kDim + 32 * half + 4 * j4);
        v[4 * j4] *= ar * g4.x; v[4 * j4 + 1] *= ar * g4.y; v[4 * j4 + 2] *= ar * g4.z; v[4 * j4 + 3] *= ar * g4.w;
      }
      umma::tmem_st16(tl + cS + 64 * (J + 1) + 32 * half, v);
      umma::tmem_st16(tl + cS + 64 * (J + 1) + 32 * half + 16, v + 16);
      if (J + 2 < kNSub) {
        umma::tmem_st16(tl + cTs + 32 * half, v);
        umma::tmem_st16(tl + cTs + 32 * half + 16, v + 16);
      }
      umma::tmem_st_wait();
      }
      umma::fence_async_smem();      // (J == 0: the P / Z diagonal blocks written above)
      sync_all();
    }
    if (s_fail) break;
    PROF(4);

    // ---- the four sub-blocks in reverse, software-pipelined: iteration I publishes the S0 / R~
    //      tiles of block I and issues its MMAs, then finishes block I+1 while they run ----------
#pragma unroll 1
    for (int I = kNSub - 1; I >= -1; --I) {
      if (I >= 0) {
        const int r0 = kSub * I;
        if (worker) {
          // lanes A: S[I];  lanes B: dOt Qt^T of block I+1 (the part of R that block added)
          float v[32];
          umma::tmem_ld16(tl + cS + 64 * I + 32 * half, *reinterpret_cast<float(*)[16]>(v));
          umma::tmem_ld16(tl + cS + 64 * I + 32 * half + 16, *reinterpret_cast<float(*)[16]>(v + 16));
          umma::tmem_ld_wait();
          if (side) {
            const float ar = aI[I * kDim + feat];
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const float4 g4 = *reinterpret_cast<const float4 *>(gI + I * kDim + 32 * half + 4 * j4);
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
          unsigned char *th = sm + (side ? oR : oS);
#pragma unroll
          for (int j8 = 0; j8 < 4; ++j8)
            write8<kTile>(th, umma::tile16_off(feat, 32 * half + 8 * j8, kDim), v + 8 * j8);
        }
        umma::fence_async_smem();
        sync_all();
        PROF(5);
        if (issuer) {
          const int cres = (I & 1) ? cTs : cRes0, cdg = (I & 1) ? cPZ : cDg0;
          const uint32_t zI = aZ + I * 2 * kTileS, pI = aP + I * 2 * kTileS;
          if (iw == 0) {
            // dOt Qt^T of this block first: the next (earlier) sub-block needs it soonest
            if (I > 0)
              gemm3<false, false, kDim, kDim, 1, kDim, false>(dB + cS + 64 * (I - 1), dlo<false, kDim>(aO, 0, I),
                                                              dlo<false, kDim>(aQ, 0, I));
            // TQ = S0^T dOt + Kt Z^T ;  T2 = Qt Z
            gemm3<true, true, kDim, kDim, 4, kSub, false>(dA + cres, dlo<true, kDim>(aS, 0, 0), dlo<true, kDim>(aO, r0, 0));
            gemm3<false, false, kDim, kSub, 1, kSub, true>(dA + cres, dlo<false, kDim>(aK, 0, I), dlo<false, kSub>(zI, 0, 0));
            gemm3<false, true, kDim, kSub, 1, kSub, false>(dA + cres + 16, dlo<false, kDim>(aQ, 0, I), dlo<true, kSub>(zI, 0, 0));
          } else if (iw == 1) {
            // T7 = R~^T Xt ;  diag(R~^T S0): boundary term of the k side
            gemm3<true, true, kDim, kDim, 4, kSub, false>(dA + cres + 32, dlo<true, kDim>(aR, 0, 0), dlo<true, kDim>(aX, r0, 0));
            gemm3<true, true, kDim, kDim, 4, kDim, false>(dA + cdg, dlo<true, kDim>(aR, 0, 0), dlo<true, kDim>(aS, 0, 0));
          } else if (iw == 2) {
            // TO = S0 Qt + Xt P^T ;  T4 = dOt P
            gemm3<false, true, kDim, kDim, 4, kSub, false>(dB + cres, dlo<false, kDim>(aS, 0, 0), dlo<true, kDim>(aQ, r0, 0));
            gemm3<false, false, kDim, kSub, 1, kSub, true>(dB + cres, dlo<false, kDim>(aX, 0, I), dlo<false, kSub>(pI, 0, 0));
            gemm3<false, true, kDim, kSub, 1, kSub, false>(dB + cres + 16, dlo<false, kDim>(aO, 0, I), dlo<true, kSub>(pI, 0, 0));
          } else {
            // T8 = R~ Kt ;  diag(S0 R~^T): boundary term of the d side
            gemm3<false, true, kDim, kDim, 4, kSub, false>(dB + cres + 32, dlo<false, kDim>(aR, 0, 0), dlo<true, kDim>(aK, r0, 0));
            gemm3<false, false, kDim, kDim, 4, kDim, false>(dB + cdg, dlo<false, kDim>(aS, 0, 0), dlo<false, kDim>(aR, 0, 0));
          }
          umma::mma_commit(&barM);
        }
        PROF(6);

        // ---- exact gate gradients of block I where the gate is too small for the cancelling
        //      form (needs only the tiles, so it runs under the MMAs):
        //   dg_t[k] = (1/g_t) sum_d M[d] N[d],  M = S0[d][k] + sum_{i<t} Xt_i[d] Kt_i[k],
        //                                       N = R~[d][k] + sum_{s>=t} dOt_s[d] Qt_s[k]
        if (worker) {
          const int n_fix = fix_n[I] < kFixCap ? fix_n[I] : kFixCap;
          for (int e = warp; e < n_fix; e += kT / 32) {
            const int code = fix_code[I * kFixCap + e];
            const int ds = code >> 16, t = (code >> 8) & 0xff, col = code & 0xff;
            // k-side entry: the fixed feature is a column of S0 / R~, X and dO rows vary with the
            // lane, the K and Q rows of the fixed feature are shared; d side: roles exchanged
            const unsigned char *var1 = sm + (ds ? oK : oX), *var2 = sm + (ds ? oQ : oO);
            const unsigned char *fix1 = sm + (ds ? oX : oK), *fix2 = sm + (ds ? oO : oQ);
            float b1[16], b2[16];
            read8(fix1, umma::tile16_off(col, r0, kDim), b1);
            read8(fix1, umma::tile16_off(col, r0 + 8, kDim), b1 + 8);
            read8(fix2, umma::tile16_off(col, r0, kDim), b2);
            read8(fix2, umma::tile16_off(col, r0 + 8, kDim), b2 + 8);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              b1[i] = (i < t) ? b1[i] : 0.f;
              b2[i] = (i >= t) ? b2[i] : 0.f;
            }
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int o = lane + 32 * j;
              float a1[16], a2[16];
              read8(var1, umma::tile16_off(o, r0, kDim), a1);
              read8(var1, umma::tile16_off(o, r0 + 8, kDim), a1 + 8);
              read8(var2, umma::tile16_off(o, r0, kDim), a2);
              read8(var2, umma::tile16_off(o, r0 + 8, kDim), a2 + 8);
              float M = ds ? rd1(sm + oS, col, o) : rd1(sm + oS, o, col);
              float N = ds ? rd1(sm + oR, col, o) : rd1(sm + oR, o, col);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                M = fmaf(a1[i], b1[i], M);
                N = fmaf(a2[i], b2[i], N);
              }
              acc = fmaf(M, N, acc);
            }
            acc = warp_sum(acc);
            if (lane == 0) fix_val[(I & 1) * kFixCap + e] = acc * fix_rg[I * kFixCap + e];
          }
        }
        PROF(7);
      }

      if (I < kNSub - 1) {
        // ---- feature-major epilogue of block J = I + 1: this thread = one feature, 8 steps -------
        const int J = I + 1, r0 = kSub * J;
        const int cres = (J & 1) ? cTs : cRes0, cdg = (J & 1) ? cPZ : cDg0;
        if (worker) {
          float r0v[8], r1v[8], r2v[8], dg[16];
          umma::tmem_ld8(tl + cres + 8 * half, r0v);
          umma::tmem_ld8(tl + cres + 16 + 8 * half, r1v);
          umma::tmem_ld8(tl + cres + 32 + 8 * half, r2v);
          umma::tmem_ld16(tl + cdg + 16 * qd, dg);
          umma::tmem_ld_wait();
          float c4 = 0.f;
#pragma unroll
          for (int e = 0; e < 16; ++e) c4 = (e == fl) ? dg[e] : c4;

          const int t0 = r0 + 8 * half;
          float mr[8], dr[8], p[8];
          const int off = umma::tile16_off(feat, t0, kDim);
          read8(mulT, off, mr);
          read8(divT, off, dr);
#pragma unroll
          for (int j = 0; j < 8; ++j) p[j] = J == 0 ? pr[0][j] : J == 1 ? pr[1][j] : J == 2 ? pr[2][j] : pr[3][j];
          const float pprev0 = J == 0 ? pp0[0] : J == 1 ? pp0[1] : J == 2 ? pp0[2] : pp0[3];
          float o1[8], o2[8], rg[8], V[8], B3[8], pre[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            o1[j] = p[j] * r0v[j];
            rg[j] = __fdividef(1.f, p[j]);
            o2[j] = (r1v[j] + r2v[j]) * rg[j];
            V[j] = mr[j] * r0v[j] - dr[j] * r1v[j];
            B3[j] = dr[j] * r2v[j];
          }
#pragma unroll
          for (int j = 6; j >= 0; --j) V[j] += V[j + 1];          // inclusive suffix over my 8 steps
          float run = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) { pre[j] = run; run += B3[j]; }   // exclusive prefix
          xc[threadIdx.x] = V[0];
          xc[kT + threadIdx.x] = run;
          umma::named_barrier(1 + qd, 64);       // the two warps that share this feature quarter
          const float oV = xc[threadIdx.x ^ 128], oB = xc[kT + (threadIdx.x ^ 128)];
          const float addV = half ? 0.f : oV;    // steps 8..15 lie after steps 0..7
          const float addB = half ? oB : 0.f;
          T *s1 = stg + (side ? 3 : 1) * kSub * kStgLd, *s2 = stg + (side ? 4 : 2) * kSub * kStgLd;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float H = V[j] + addV + pre[j] + addB + c4;
            const float pprev = j ? p[j - 1] : pprev0;
            const int lr = 8 * half + j;
            if (!side) stg[lr * kStgLd + feat] = (T)o1[j];
            s1[lr * kStgLd + feat] = (T)o2[j];
            s2[lr * kStgLd + feat] = (T)(H * pprev * rg[j]);
          }
        }
        sync_all();     // staging complete
        PROF(8);
        const int n_fix = fix_n[J] < kFixCap ? fix_n[J] : kFixCap;
        if (n_fix > 0) {
          if (threadIdx.x < n_fix) {
            const int code = fix_code[J * kFixCap + threadIdx.x];
            const int ds = code >> 16, t = (code >> 8) & 0xff, col = code & 0xff;
            stg[((ds ? 4 : 2) * kSub + t) * kStgLd + col] = (T)fix_val[(J & 1) * kFixCap + threadIdx.x];
          }
          __syncthreads();
        }
        // ---- coalesced write of the five 16 x 64 result tiles ----------------------------------
        if (worker) {
          T *dst[5] = {dq, dk, dfk, dx, df};
          for (int idx = threadIdx.x; idx < 5 * kSub * 8; idx += kT) {
            const int it = idx >> 7, r = (idx >> 3) & 15, ch = idx & 7;
            if (r0 + r < nvalid) {
              const uint4 val = *reinterpret_cast<const uint4 *>(stg + (it * kSub + r) * kStgLd + ch * 8);
              *reinterpret_cast<uint4 *>(dst[it] + base + (size_t)(r0 + r) * kDim + ch * 8) = val;
            }
          }
        }
        PROF(9);
      }

      if (I >= 0) wait_mma();     // the MMAs of block I
      sync_all();                 // also: everything of block I+1 consumed
      PROF(10);
      if (s_fail) break;
    }
    if (s_fail) break;
  }
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
    lfw_chunk_bwd_umma_kernel<TT><<<grid, kTAll, kSmem, st>>>(                                           \
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
