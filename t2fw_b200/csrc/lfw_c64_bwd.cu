// Sequence gradients of the chunked decay-rule backward on the tcgen05 tensor core (D = K = 64,
// 16-bit storage, chunks of 64 steps): d_x, d_f, d_q, d_k, d_f_key of one chunk from its inputs,
// the state at the chunk start (checkpoint) and the state gradient at the chunk end (carried over
// the chunks by lfw_chunk_bwd_carry_kernel).  Replaces the reference's reverse scan, its
// materialised state gradients, five einsums and two in-place multiplies
// (t2fw/csrc/lfw_kernel.cu:61-102, t2fw/csrc/lfw.cpp:84-93).
//
// The k side (d_q, d_k, d_f_key) and the d side (d_x, d_f) are mirror images, so one code path
// runs twice per chunk with the roles exchanged ("own" side = the side whose gradients are
// formed, "other" side = the side that is contracted away).  For the k side (own = k, other = d;
// notation of lfw_c64.cuh, S0 = start state, R = end state gradient, both viewed [own][other]):
//     Z    = tril( (dO pm_a) (x / pm_a)^T )                              [t][s], in-chunk decays of the other side
//     TQ   = (G_REF .* S0) (dO A_t)^T  +  (k / pm_g) Z^T                 [k][t]
//     T2   = (q pm_g) Z                                                  [k][s]
//     T7   = (G_63/G_REF .* R) (x A_63/A_s)^T                            [k][s]
//     d_q  = pm_g .* TQ          d_k = (T2 + T7) ./ pm_g
//     g_t d_g_t = sum_{s>=t} [(q pm_g) .* TQ - (k / pm_g) .* T2]_s + sum_{i<t} [(k / pm_g) .* T7]_i
//                 + G_63 .* sum_d A_63 S0 R                              (d_f_key = that / g_t)
// The suffix sum cancels the pair terms (i, s >= t) of its two parts; both parts come from the same
// TF32-rounded Z and operands, so the cancellation is exact up to fp32 accumulation.  Where a gate
// is below 2^-10 even that is not enough (the result is divided by the gate), and the pair terms
// i < t <= s are summed directly for that (t, feature).
// Results are feature-major ([own feature][step], rows = tensor-memory lanes): after tcgen05.ld a
// thread owns one feature over eight steps, so the sums over time are register-local plus one
// exchange between the eight threads of a feature.
//
// One persistent CTA of 16 warps per SM; six raw 8 KB input blocks per chunk by bulk asynchronous
// copy (the next chunk's are requested as soon as the second pass has consumed this chunk's);
// operand tiles in shared memory (TF32, 128-byte swizzle), accumulators in tensor memory, MMAs
// issued by four elected threads.
#include <type_traits>

#include "lfw_c64.cuh"

namespace t2fw {

using namespace c64;

int lfw_chunk_status_ptr(int **out);   // lfw_chunk_local_umma.cu

#ifdef T2FW_C64_PROFILE
__device__ long long g_c64_prof[32];
#define PROF(i)                                                    \
  do {                                                             \
    if (threadIdx.x == 96 && blockIdx.x == 0) {                    \
      const long long now_ = clock64();                            \
      g_c64_prof[i] += now_ - tprev;                               \
      tprev = now_;                                                \
    }                                                              \
  } while (0)
#else
#define PROF(i) do { } while (0)
#endif

namespace {

constexpr int kThreadsB = 512;
constexpr int kPmLd = 68;              // row stride (floats) of the own-side ratio table
constexpr int kFixCap = 128;           // tiny-gate entries per pass
// shared-memory map (bytes from the 1024-byte aligned base)
//   tiles: 0 Mo_mid -> Z[t][s]   1 Vo_mid -> Z^T[s][t]   2 Mo_start   3 Vo_end
//          4 Vw_mid [own][t]     5 Mw_mid [own][t]       6 S2 [own][other]              7 R2 [own][other]
constexpr int oT = 0;
constexpr int oPm = oT + 8 * kTile;                 // pm_w[own][t]   (ratios of the own side)
constexpr int oPmo = oPm + kDim * kPmLd * 4;        // pm_o[t][other] (ratios of the other side)
constexpr int oQt = oPmo + kC * kDim * 4;           // quarter products [other, own][4][64]
constexpr int oXc = oQt + 2 * 4 * kDim * 4;         // partial sums [3][8 ranges][64]
constexpr int oBnd = oXc + 3 * 8 * kDim * 4;        // boundary-term partials [8][64]
constexpr int oFixCode = oBnd + 8 * kDim * 4;       // [kFixCap] int
constexpr int oFixVal = oFixCode + kFixCap * 4;     // [kFixCap] float
constexpr int oFixMask = oFixVal + kFixCap * 4;     // [64] one bit per step
constexpr int oRaw = oFixMask + kDim * 8;           // x, f, q, k, fk, dO
constexpr int kSmemB = oRaw + 6 * kRawBytes + 1024; // + slack for the 1024-byte alignment
static_assert(oRaw % 128 == 0 && oFixMask % 8 == 0, "alignment");
static_assert(kSmemB + 128 <= 227 * 1024, "shared memory limit");

constexpr int cZ = 0, cTQ1 = 32, cTQ2 = 64, cT2 = 96, cT7 = 128;   // tensor-memory columns
constexpr int kTmemCols = 256;

template <typename T>
__global__ void __launch_bounds__(kThreadsB, 1)
lfw_c64_bwd_kernel(const T *__restrict__ go, const T *__restrict__ x, const T *__restrict__ f,
                   const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ fk,
                   const T *__restrict__ state, const T *__restrict__ ckpt, const float *__restrict__ Rend,
                   T *__restrict__ dx, T *__restrict__ df, T *__restrict__ dq, T *__restrict__ dk,
                   T *__restrict__ dfk, int *__restrict__ rowflag, int *__restrict__ status, int64_t T_,
                   int64_t nc, int64_t total) {
  extern __shared__ __align__(1024) unsigned char sm_raw[];
  unsigned char *sm = sm_raw + ((1024u - (umma::smem_u32(sm_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t barRaw, barZ, barM;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail, s_bad, fix_n;

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  // stage 1: 0 = other side, 1 = own side; 16-step quarter; feature
  const int gsw = warp >> 3, tq = (warp >> 1) & 3, feat = (warp & 1) * 32 + lane;
  // accumulator read-out: lane quarter, column part, lane set, row inside the quarter
  const int q4 = warp & 3, part = warp >> 2, h = lane >> 4, fl = lane & 15;
  // state tiles: own row, eight other columns
  const int sr = tid & 63, sc0 = (tid >> 6) * 8;

  float *pmT = reinterpret_cast<float *>(sm + oPm);
  float *pmo = reinterpret_cast<float *>(sm + oPmo);
  float *qtot = reinterpret_cast<float *>(sm + oQt);
  float *xc = reinterpret_cast<float *>(sm + oXc);
  float *bndp = reinterpret_cast<float *>(sm + oBnd);
  int *fix_code = reinterpret_cast<int *>(sm + oFixCode);
  float *fix_val = reinterpret_cast<float *>(sm + oFixVal);
  unsigned long long *fix_mask = reinterpret_cast<unsigned long long *>(sm + oFixMask);
  T *raw = reinterpret_cast<T *>(sm + oRaw);     // [6][64][64]: x, f, q, k, fk, dO

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

  if (tid == 0) {
    umma::mbar_init(&barRaw, 1);
    umma::mbar_init(&barZ, 2);
    umma::mbar_init(&barM, 6);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, kTmemCols);
  sync_all();
  const uint32_t tb = __shfl_sync(0xffffffffu, tmem_slot, 0);
  const uint32_t tl = umma::tmem_addr(tb, 32 * q4, 0);
  bool raw_pending = false;      // thread 0
  if (tid == 0 && (int64_t)blockIdx.x < total) {
    issue_raw(blockIdx.x);
    raw_pending = true;
  }
  const uint32_t aT = umma::smem_u32(sm + oT);
  uint64_t dT[8];      // descriptors of the eight tiles
#pragma unroll
  for (int i = 0; i < 8; ++i) dT[i] = desc_sw128(aT + i * kTile);
  uint32_t pz = 0, pm_par = 0;   // mbarrier phase parities

#ifdef T2FW_C64_PROFILE
  long long tprev = clock64();
#endif
  uint32_t it = 0;
  for (int64_t ci = blockIdx.x; ci < total; ci += gridDim.x, ++it) {
    const int64_t b = ci / nc, c = ci % nc, t0c = c * kC;
    const int nvalid = (int)((T_ - t0c < kC) ? T_ - t0c : kC);
    PROF(0);
    const size_t base = ((size_t)b * T_ + t0c) * kDim;
    const T *s0p = (c == 0) ? state + (size_t)b * kDim * kDim : ckpt + ((size_t)b * nc + (c - 1)) * kDim * kDim;
    const float *rp = Rend + (size_t)ci * kDim * kDim;

    if (!acp::mbar_wait(&barRaw, it & 1u)) s_fail = 1;
    if (tid == 0) raw_pending = false;
    __syncthreads();
    if (s_fail) break;
    if (nvalid < kC) {      // partial chunk: identity steps beyond the valid ones
      pad_raw_tail<T>(raw, 6, (1u << 1) | (1u << 4), nvalid, tid, kThreadsB);
      __syncthreads();
    }
    PROF(1);

#pragma unroll 1
    for (int ph = 0; ph < 2; ++ph) {
      // pass 0: own = k side (other = d side);  pass 1: own = d side
      const int blk_go = ph ? 4 : 1, blk_mo = ph ? 2 : 5, blk_vo = ph ? 3 : 0;   // other: gate, mul, div
      const int blk_gw = ph ? 1 : 4, blk_mw = ph ? 5 : 2, blk_vw = ph ? 0 : 3;   // own
      // ---- start state and end gradient as S(own = sr, other = sc0 + j): requested now, converted
      //      when they are used ----
      unsigned short s16[8];     // pass 0: one 16-bit value per register (nothing depends on the loads yet)
      uint4 s4 = make_uint4(0u, 0u, 0u, 0u);     // pass 1: eight packed values
      float rv[8];
      if (ph == 0) {
        const unsigned short *s0u = reinterpret_cast<const unsigned short *>(s0p);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s16[j] = s0u[(sc0 + j) * kDim + sr];
          rv[j] = rp[(sc0 + j) * kDim + sr];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) s16[j] = 0;
        s4 = *reinterpret_cast<const uint4 *>(s0p + sr * kDim + sc0);
        const float4 r0 = *reinterpret_cast<const float4 *>(rp + sr * kDim + sc0);
        const float4 r1 = *reinterpret_cast<const float4 *>(rp + sr * kDim + sc0 + 4);
        rv[0] = r0.x; rv[1] = r0.y; rv[2] = r0.z; rv[3] = r0.w;
        rv[4] = r1.x; rv[5] = r1.y; rv[6] = r1.z; rv[7] = r1.w;
      }

      // ---- stage 1: gate products of the four quarters, then the ratios to the anchor ----
      if (tid == 0) {
        s_bad = 0;
        fix_n = 0;
      }
      if (tid < kDim) fix_mask[tid] = 0ull;
      float g[16];
      qtot[(gsw * 4 + tq) * kDim + feat] = load_gates16<T>(raw + (gsw ? blk_gw : blk_go) * kC * kDim + feat, tq, g);
      __syncthreads();
      PROF(2);
      {
        const float *qt = qtot + gsw * 4 * kDim + feat;
        const float carry = tq == 0 ? qt[kDim] : tq == 3 ? qt[2 * kDim] : 1.f;
        float pm[16];
        if (!ratios16(tq, g, carry, pm)) s_bad = 1;
        if (gsw == 0) {
#pragma unroll
          for (int j = 0; j < 16; ++j) pmo[(16 * tq + j) * kDim + feat] = pm[j];
        } else {
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<float4 *>(pmT + feat * kPmLd + 16 * tq + j) = make_float4(pm[j], pm[j + 1], pm[j + 2], pm[j + 3]);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (fabsf(g[j]) < kTinyGate && 16 * tq + j < nvalid) {   // exact pair sum for this (step, feature) later
              const int slot = atomicAdd(&fix_n, 1);
              if (slot < kFixCap) {
                fix_code[slot] = ((16 * tq + j) << 8) | feat;
                atomicOr(&fix_mask[feat], 1ull << (16 * tq + j));
              } else {
                s_bad = 1;
              }
            }
          }
        }
      }
      __syncthreads();
      PROF(3);

      // ---- stage 2: operand tiles ----
      {   // other side, time-major: this thread = four features, steps t and t + 32
        const int f4 = (tid & 15) * 4;
        const float4 o_ref = mul4(*reinterpret_cast<const float4 *>(qtot + f4),
                                  *reinterpret_cast<const float4 *>(qtot + kDim + f4));
        const float4 oc_ref = mul4(*reinterpret_cast<const float4 *>(qtot + 2 * kDim + f4),
                                   *reinterpret_cast<const float4 *>(qtot + 3 * kDim + f4));
        const T *r_m = raw + blk_mo * kC * kDim + f4, *r_v = raw + blk_vo * kC * kDim + f4;
        unsigned char *t0p = sm + oT;
#pragma unroll
        for (int i2 = 0; i2 < 2; ++i2) {
          const int t = (tid >> 4) + 32 * i2;
          const float4 pv = *reinterpret_cast<const float4 *>(pmo + t * kDim + f4);
          const float4 m = mul4(Vec4<T>::ld(r_m + t * kDim), pv);
          const float4 v = mul4(Vec4<T>::ld(r_v + t * kDim), rcp4(pv));
          const int o = toff(t, f4);
          *reinterpret_cast<float4 *>(t0p + o) = rna4(m);
          *reinterpret_cast<float4 *>(t0p + kTile + o) = rna4(v);
          *reinterpret_cast<float4 *>(t0p + 2 * kTile + o) = rna4(mul4(m, o_ref));
          *reinterpret_cast<float4 *>(t0p + 3 * kTile + o) = rna4(mul4(v, oc_ref));
        }
      }
      {   // own side, feature-major: this thread = features 2 * lane, 2 * lane + 1, steps 4 * warp .. + 3
        const int f0 = 2 * lane, t = 4 * warp;
        const T *r_m = raw + blk_mw * kC * kDim + t * kDim + f0, *r_v = raw + blk_vw * kC * kDim + t * kDim + f0;
        float2 m2[4], v2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          m2[j] = Vec2<T>::ld(r_m + j * kDim);
          v2[j] = Vec2<T>::ld(r_v + j * kDim);
        }
        const float4 p0 = *reinterpret_cast<const float4 *>(pmT + f0 * kPmLd + t);
        const float4 p1 = *reinterpret_cast<const float4 *>(pmT + (f0 + 1) * kPmLd + t);
        const float4 i0 = rcp4(p0), i1 = rcp4(p1);
        unsigned char *t4p = sm + oT + 4 * kTile, *t5p = sm + oT + 5 * kTile;
        const int o0 = toff(f0, t), o1 = toff(f0 + 1, t);
        *reinterpret_cast<float4 *>(t5p + o0) = rna4(mul4(make_float4(m2[0].x, m2[1].x, m2[2].x, m2[3].x), p0));
        *reinterpret_cast<float4 *>(t5p + o1) = rna4(mul4(make_float4(m2[0].y, m2[1].y, m2[2].y, m2[3].y), p1));
        *reinterpret_cast<float4 *>(t4p + o0) = rna4(mul4(make_float4(v2[0].x, v2[1].x, v2[2].x, v2[3].x), i0));
        *reinterpret_cast<float4 *>(t4p + o1) = rna4(mul4(make_float4(v2[0].y, v2[1].y, v2[2].y, v2[3].y), i1));
      }
      PROF(14);
      // ---- state tiles S2 = W_REF .* S0, R2 = W_63/W_REF .* R, boundary partial sums ----
      {
        const float w_ref = qtot[4 * kDim + sr] * qtot[5 * kDim + sr];
        const float wc_ref = qtot[6 * kDim + sr] * qtot[7 * kDim + sr];
        float s2[8], r2[8], acc = 0.f;
        if (ph) {
          s16[0] = (unsigned short)s4.x; s16[1] = (unsigned short)(s4.x >> 16);
          s16[2] = (unsigned short)s4.y; s16[3] = (unsigned short)(s4.y >> 16);
          s16[4] = (unsigned short)s4.z; s16[5] = (unsigned short)(s4.z >> 16);
          s16[6] = (unsigned short)s4.w; s16[7] = (unsigned short)(s4.w >> 16);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int o = sc0 + j;
          const float oc = (qtot[o] * qtot[kDim + o]) * (qtot[2 * kDim + o] * qtot[3 * kDim + o]);
          s2[j] = rna_tf32(Elem<T>::ld(reinterpret_cast<const T *>(&s16[j])) * w_ref);
          r2[j] = rna_tf32(rv[j] * wc_ref);
          acc = fmaf(oc * s2[j], r2[j], acc);
        }
        unsigned char *t6p = sm + oT + 6 * kTile, *t7p = sm + oT + 7 * kTile;
        const int o0 = toff(sr, sc0), o1 = toff(sr, sc0 + 4);
        *reinterpret_cast<float4 *>(t6p + o0) = make_float4(s2[0], s2[1], s2[2], s2[3]);
        *reinterpret_cast<float4 *>(t6p + o1) = make_float4(s2[4], s2[5], s2[6], s2[7]);
        *reinterpret_cast<float4 *>(t7p + o0) = make_float4(r2[0], r2[1], r2[2], r2[3]);
        *reinterpret_cast<float4 *>(t7p + o1) = make_float4(r2[4], r2[5], r2[6], r2[7]);
        bndp[(tid >> 6) * kDim + sr] = acc;
      }
      PROF(4);
      umma::fence_async_smem();
      sync_all();       // tiles complete; in the second pass the raw blocks are consumed
      PROF(5);

      // ---- first MMA round: one issuing thread per 32-column half ----
      if (warp < 2) {
        const uint32_t dh = umma::tmem_addr(tb, 16 * warp, 0);
        if (elect_one()) {
          mma_64x32x64(dh + cZ, dT[0], dT[1], 32 * warp, false);        // Z = Mo_mid Vo_mid^T
          umma::mma_commit(&barZ);
          mma_64x32x64(dh + cTQ1, dT[6], dT[2], 32 * warp, false);      // TQ1 = S2 Mo_start^T
          mma_64x32x64(dh + cT7, dT[7], dT[3], 32 * warp, false);       // T7 = R2 Vo_end^T
          umma::mma_commit(&barM);
        }
        __syncwarp();
        if (tid == 0) {
          if (s_bad) atomicExch(rowflag + b, 1);      // the scan kernels redo this batch row
          if (ph == 1 && ci + gridDim.x < total) {
            issue_raw(ci + gridDim.x);
            raw_pending = true;
          }
        }
      }

      // ---- Z: mask, round, store as [t][s] (tile 0) and [s][t] (tile 1) ----
      if (!umma::mbar_wait(&barZ, pz)) s_fail = 1;
      pz ^= 1u;
      umma::fence_after_sync();
      PROF(6);
      {
        const int t = 16 * q4 + fl, s0 = 32 * h + 8 * part;
        float v[8];
        umma::tmem_ld8(tl + cZ + 8 * part, v);
        umma::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (s0 + j <= t) ? rna_tf32(v[j]) : 0.f;
        unsigned char *t0p = sm + oT, *t1p = t0p + kTile;
        *reinterpret_cast<float4 *>(t0p + toff(t, s0)) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(t0p + toff(t, s0 + 4)) = make_float4(v[4], v[5], v[6], v[7]);
#pragma unroll
        for (int j = 0; j < 8; ++j) *reinterpret_cast<float *>(t1p + toff(s0 + j, t)) = v[j];
      }
      PROF(7);
      umma::fence_async_smem();
      sync_all();
      if (s_fail) break;
      PROF(8);

      // ---- second MMA round: TQ2 = Vw_mid Z^T (warps 0, 1), T2 = Mw_mid Z (warps 2, 3) ----
      if (warp < 4) {
        const int hh = warp & 1;
        const uint32_t dh = umma::tmem_addr(tb, 16 * hh, 0);
        if (elect_one()) {
          if (warp < 2) mma_64x32x64(dh + cTQ2, dT[4], dT[0], 32 * hh, false);
          else mma_64x32x64(dh + cT2, dT[5], dT[1], 32 * hh, false);
          umma::mma_commit(&barM);
        }
        __syncwarp();
      }
      // ---- tiny gates: pair terms i < t <= s summed directly (runs under the MMAs) ----
      {
        const int n_fix = fix_n < kFixCap ? fix_n : kFixCap;
        const unsigned char *zt = sm + oT, *vw = sm + oT + 4 * kTile, *mw = sm + oT + 5 * kTile;
        for (int e = warp; e < n_fix; e += kThreadsB / 32) {
          const int code = fix_code[e], t = code >> 8, own = code & 0xff;
          // sum_{s >= t} Mw[s] sum_{i < t} Z[s][i] Vw[i]: lanes over i, independent loads over s
          float acc = 0.f;
          for (int i = lane; i < t; i += 32) {
            float a = 0.f;
#pragma unroll 8
            for (int s = t; s < kC; ++s)
              a = fmaf(*reinterpret_cast<const float *>(mw + toff(own, s)),
                       *reinterpret_cast<const float *>(zt + toff(s, i)), a);
            acc = fmaf(a, *reinterpret_cast<const float *>(vw + toff(own, i)), acc);
          }
          acc = warp_sum(acc);
          if (lane == 0) fix_val[e] = acc;
        }
      }
      PROF(9);
      __syncthreads();      // fix_val, bndp visible
      PROF(10);

      // ---- feature-major epilogue: this thread = one own feature, 8 steps ----
      {
        const int own = 16 * q4 + fl, t0e = 32 * h + 8 * part, ridx = 4 * h + part;
        float mw[8], vw[8], pmv[9];
        {
          const unsigned char *t4p = sm + oT + 4 * kTile, *t5p = sm + oT + 5 * kTile;
          const float4 a0 = *reinterpret_cast<const float4 *>(t5p + toff(own, t0e));
          const float4 a1 = *reinterpret_cast<const float4 *>(t5p + toff(own, t0e + 4));
          const float4 b0 = *reinterpret_cast<const float4 *>(t4p + toff(own, t0e));
          const float4 b1 = *reinterpret_cast<const float4 *>(t4p + toff(own, t0e + 4));
          mw[0] = a0.x; mw[1] = a0.y; mw[2] = a0.z; mw[3] = a0.w; mw[4] = a1.x; mw[5] = a1.y; mw[6] = a1.z; mw[7] = a1.w;
          vw[0] = b0.x; vw[1] = b0.y; vw[2] = b0.z; vw[3] = b0.w; vw[4] = b1.x; vw[5] = b1.y; vw[6] = b1.z; vw[7] = b1.w;
          const float4 p0 = *reinterpret_cast<const float4 *>(pmT + own * kPmLd + t0e);
          const float4 p1 = *reinterpret_cast<const float4 *>(pmT + own * kPmLd + t0e + 4);
          pmv[1] = p0.x; pmv[2] = p0.y; pmv[3] = p0.z; pmv[4] = p0.w; pmv[5] = p1.x; pmv[6] = p1.y; pmv[7] = p1.z; pmv[8] = p1.w;
          // ratio of the step before this range; before step 0 it is 1 / W_REF
          pmv[0] = t0e ? pmT[own * kPmLd + t0e - 1]
                       : __fdividef(1.f, qtot[4 * kDim + own] * qtot[5 * kDim + own]);
        }
        float bnd = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) bnd += bndp[r * kDim + own];
        const unsigned m8 = (unsigned)((fix_mask[own] >> t0e) & 0xffull);
        float gr[8], ip[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ip[j] = __fdividef(1.f, pmv[j + 1]);
          gr[j] = pmv[j] * ip[j];                       // 1 / gate
        }
        if (!umma::mbar_wait(&barM, pm_par)) s_fail = 1;
        pm_par ^= 1u;
        umma::fence_after_sync();
        PROF(11);
        float tq1[8], tq2[8], t2v[8], t7v[8];
        umma::tmem_ld8(tl + cTQ1 + 8 * part, tq1);
        umma::tmem_ld8(tl + cTQ2 + 8 * part, tq2);
        umma::tmem_ld8(tl + cT2 + 8 * part, t2v);
        umma::tmem_ld8(tl + cT7 + 8 * part, t7v);
        umma::tmem_ld_wait();
        float dmu[8], ddv[8], sa[8], sb[8], pre[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dmu[j] = pmv[j + 1] * (tq1[j] + tq2[j]);
          ddv[j] = (t2v[j] + t7v[j]) * ip[j];
          sa[j] = mw[j] * tq1[j];
          sb[j] = mw[j] * tq2[j] - vw[j] * t2v[j];
          pre[j] = vw[j] * t7v[j];
        }
#pragma unroll
        for (int j = 6; j >= 0; --j) { sa[j] += sa[j + 1]; sb[j] += sb[j + 1]; }   // inclusive suffix sums
        float run = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float v = pre[j]; pre[j] = run; run += v; }   // exclusive prefix
        xc[(0 * 8 + ridx) * kDim + own] = sa[0];
        xc[(1 * 8 + ridx) * kDim + own] = sb[0];
        xc[(2 * 8 + ridx) * kDim + own] = run;
        umma::named_barrier(1 + q4, 128);       // the four warps that share this lane quarter
        float addA = 0.f, addB = 0.f, addP = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float va = xc[(0 * 8 + r) * kDim + own], vb2 = xc[(1 * 8 + r) * kDim + own];
          const float vp = xc[(2 * 8 + r) * kDim + own];
          addA += (r > ridx) ? va : 0.f;        // later steps
          addB += (r > ridx) ? vb2 : 0.f;
          addP += (r < ridx) ? vp : 0.f;        // earlier steps
        }
        const float base_h = addA + addP + bnd;
#pragma unroll
        for (int j = 0; j < 8; ++j) sb[j] += addB;
        if (m8) {        // some gate of this range is tiny: its pair terms were summed directly
          const int n_fix = fix_n < kFixCap ? fix_n : kFixCap;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if ((m8 >> j) & 1u)
              for (int e = 0; e < n_fix; ++e)
                if (fix_code[e] == (((t0e + j) << 8) | own)) sb[j] = fix_val[e];
        }
        // 16 consecutive features of one step are 32 contiguous bytes: the results go straight out
        T *o_mu = (ph ? nullptr : dq) , *o_dv = ph ? dx : dk, *o_gt = ph ? df : dfk;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = t0e + j;
          const float H = sa[j] + sb[j] + pre[j] + base_h;
          if (t < nvalid) {
            const size_t o = base + (size_t)t * kDim + own;
            if (ph == 0) o_mu[o] = (T)dmu[j];
            o_dv[o] = (T)ddv[j];
            o_gt[o] = (T)(H * gr[j]);
          }
        }
      }
      PROF(12);
      sync_all();
      if (s_fail) break;
      PROF(13);
    }
    if (s_fail) break;
  }
  if (tid == 0) {
    if (s_fail) {
      atomicExch(status, 1);
      if (raw_pending) acp::mbar_wait(&barRaw, it & 1u);   // bounded: let the copies in flight land
    }
  }
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, kTmemCols);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int g_sms_b[64] = {};

}  // namespace

// Returns T2FW_ERR_UNSUPPORTED (without launching) if a pointer is not 16-byte aligned.
int lfw_c64_backward_main(const void *go, const void *x, const void *f, const void *q, const void *k,
                          const void *fk, const void *state, const void *ckpt, const float *Rend, void *dx,
                          void *df, void *dq, void *dk, void *dfk, int *rowflag, int64_t B, int64_t T_,
                          int dtype, cudaStream_t st) {
  if (!(aligned16(go) && aligned16(x) && aligned16(f) && aligned16(q) && aligned16(k) && aligned16(fk) &&
        aligned16(state) && aligned16(ckpt) && aligned16(Rend) && aligned16(dx) && aligned16(df) &&
        aligned16(dq) && aligned16(dk) && aligned16(dfk)))
    return T2FW_ERR_UNSUPPORTED;
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return T2FW_ERR_UNSUPPORTED;
  if (g_sms_b[dev] == 0) {
    int n = 0;
    T2FW_CHECK_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    g_sms_b[dev] = n;
  }
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  const int64_t nc = ceil_div64(T_, kC), total = B * nc;
  const unsigned grid = (unsigned)(total < g_sms_b[dev] ? total : g_sms_b[dev]);
#define T2FW_LAUNCH(TT)                                                                               \
  do {                                                                                                \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_c64_bwd_kernel<TT>,                                      \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemB));       \
    lfw_c64_bwd_kernel<TT><<<grid, kThreadsB, kSmemB, st>>>(                                          \
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

#ifdef T2FW_C64_PROFILE
extern "C" int t2fw_debug_c64_prof(long long *out) {
  return (int)cudaMemcpyFromSymbol(out, t2fw::g_c64_prof, sizeof(long long) * 32);
}
#endif
