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
// is below 2^-13 even that is not enough (the result is divided by the gate), and the pair terms
// i < t <= s are summed directly for that (t, feature).
// Results are feature-major ([own feature][step], rows = tensor-memory lanes): after tcgen05.ld a
// thread owns one feature over eight steps, so the sums over time are register-local plus one
// exchange between the eight threads of a feature.
//
// One persistent CTA of 16 warps per SM; six raw 8 KB input blocks per chunk by bulk asynchronous
// copy (the next chunk's are requested as soon as the second pass has consumed this chunk's);
// operand tiles in shared memory (TF32, 128-byte swizzle), accumulators in tensor memory, MMAs
// issued by one elected lane.
#include <type_traits>

#include "lfw_c64.cuh"
#include "seq_layout.cuh"

namespace t2fw {

using namespace c64;

int lfw_chunk_status_ptr(int **out);   // lfw_c64_local.cu
int lfw_chunk_sm_count(int *out);


namespace {

constexpr int kThreadsB = 512;
constexpr int kPmLd = 68;              // row stride (floats) of the own-side ratio table
constexpr int kFixCap = 128;           // tiny-gate entries per pass
constexpr int kS0Ld = 144;             // row stride (bytes) of the start-state landing zone (64 x 16-bit + pad)
constexpr int kRLd = 272;              // row stride (bytes) of the end-gradient landing zone (64 x fp32 + pad)
// shared-memory map (bytes from the 1024-byte aligned base)
//   tiles: 0 Mo_mid -> Z[t][s]   1 Vo_mid -> Z^T[s][t]   2 Mo_start   3 Vo_end     (B operands)
constexpr int oT = 0;
constexpr int oPm = oT + 4 * kTile;                 // pm_w[own][t]   (ratios of the own side)
constexpr int oPmo = oPm + kDim * kPmLd * 4;        // pm_o[t][other] (ratios of the other side)
constexpr int oQt = oPmo + kC * kDim * 4;           // quarter products [pass][other, own][4][64]
constexpr int oPrd = oQt + 2 * 2 * 4 * kDim * 4;    // products of the quarter products [pass][6][64], see the ratio stage
constexpr int oXc = oPrd + 2 * 6 * kDim * 4;        // partial sums [3][8 ranges][64]
constexpr int oBnd = oXc + 3 * 8 * kDim * 4;        // boundary-term partials [8][64]
constexpr int oFixCode = oBnd + 8 * kDim * 4;       // [kFixCap] int
constexpr int oFixVal = oFixCode + kFixCap * 4;     // [kFixCap] float
constexpr int oFixMask = oFixVal + kFixCap * 4;     // [pass][64] one bit per step
constexpr int kFixRows = 16;                        // features with tiny gates per pass whose operand rows are kept
constexpr int oFixSlot = oFixMask + 2 * kDim * 8;   // [64] int: row slot of a feature, -1 = none
constexpr int oFixRow = oFixSlot + kDim * 4;        // [kFixRows][2][64] floats: own-side operand rows Mw, Vw
constexpr int oS0L = oFixRow + kFixRows * 2 * kDim * 4;   // start state of the chunk, [64][kS0Ld]
constexpr int oRL = oS0L + kDim * kS0Ld;            // end state gradient of the chunk, [64][kRLd]
constexpr int oRaw = oRL + kDim * kRLd;             // x, f, q, k, fk, dO, and (fused layer) the gate pre-activations
constexpr int kSmemB = oRaw + 7 * kRawBytes + 1024; // + slack for the 1024-byte alignment
static_assert(oRaw % 128 == 0 && oFixMask % 8 == 0 && oS0L % 16 == 0 && oRL % 16 == 0, "alignment");
static_assert(kSmemB + 128 <= 227 * 1024, "shared memory limit");

// tensor-memory columns: the four A operands [own][64] (both lane sets), then the accumulators
constexpr int cS2 = 0, cR2 = 64, cVw = 128, cMw = 192;
constexpr int cZ = 256, cTQ1 = 288, cTQ2 = 320, cT2 = 352, cT7 = 384;
constexpr int kTmemCols = 512;

// kFused = false: the plain operator (no activation flags, query scale 1), decided at compile time.
template <typename T, bool kFused>
__global__ void __launch_bounds__(kThreadsB, 1)
lfw_c64_bwd_kernel(const __grid_constant__ seq::Maps mp, const T *__restrict__ state, const T *__restrict__ ckpt,
                   const float *__restrict__ Rend, const seq::Out<T> dx, const seq::Out<T> df, const seq::Out<T> dq,
                   const seq::Out<T> dk, const seq::Out<T> dfk, int *__restrict__ rowflag, int *__restrict__ status,
                   int64_t T_, int64_t nc, int64_t total) {
  extern __shared__ __align__(1024) unsigned char sm_raw[];
  unsigned char *sm = sm_raw + ((1024u - (umma::smem_u32(sm_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t barRaw, barZ, barM;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail, s_bad, fix_n2[2], fix_rows_n;

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  // stage 1: 0 = other side, 1 = own side; 16-step quarter; feature
  const int gsw = warp >> 3, tq = (warp >> 1) & 3, feat = (warp & 1) * 32 + lane;
  // tensor-memory rows: lane quarter, column part, lane set, row inside the quarter.  Thread
  // (q4, part, h, fl) owns row 16 * q4 + fl and the eight columns 8 * (4 * h + part) .. + 7 of the
  // own-side operands, of the state blocks and of every result.
  const int q4 = warp & 3, part = warp >> 2, h = lane >> 4, fl = lane & 15;
  const int own = 16 * q4 + fl, cg = 4 * h + part, c0 = 8 * cg;

  float *pmT = reinterpret_cast<float *>(sm + oPm);
  float *pmo = reinterpret_cast<float *>(sm + oPmo);
  float *qtot2 = reinterpret_cast<float *>(sm + oQt);
  float *prd2 = reinterpret_cast<float *>(sm + oPrd);
  float *xc = reinterpret_cast<float *>(sm + oXc);
  float *bndp = reinterpret_cast<float *>(sm + oBnd);
  int *fix_code = reinterpret_cast<int *>(sm + oFixCode);
  float *fix_val = reinterpret_cast<float *>(sm + oFixVal);
  unsigned long long *fix_mask2 = reinterpret_cast<unsigned long long *>(sm + oFixMask);
  int *fix_slot = reinterpret_cast<int *>(sm + oFixSlot);
  float *fix_rows = reinterpret_cast<float *>(sm + oFixRow);
  T *raw = reinterpret_cast<T *>(sm + oRaw);     // [6][64][64]: x, f, q, k, fk, dO

  // tensors: 0 x, 1 f, 2 q, 3 k, 4 fk, 5 dO
  const bool unit_forget = kFused && (mp.flags & seq::kUnitForget) != 0;
  const bool sigmoid_gate = kFused && (mp.flags & seq::kSigmoidGate) != 0;
  const float q_scale = kFused ? mp.q_scale : 1.f;
  auto issue_raw = [&](int64_t ci) {     // thread 0 only: one copy per tensor
    const Item w = split_item(ci, nc, mp.heads);
    const int row = (int)(w.b * T_ + w.c * kC), hc = w.h;
    const int nv = (int)((T_ - (int64_t)w.c * kC < kC) ? T_ - (int64_t)w.c * kC : kC);
    unsigned char *r = sm + oRaw;
    const uint32_t per = (mp.flags & seq::kContiguous) ? (uint32_t)nv * kDim * sizeof(T) : (uint32_t)kRawBytes;
    const bool sigm = sigmoid_gate;
    acp::mbar_expect_tx(&barRaw, ((unit_forget ? 5u : 6u) + (sigm ? 1u : 0u)) * per);
#pragma unroll
    for (int i = 0; i < 6; ++i)
      if (!(i == 1 && unit_forget)) seq::fetch_block<T>(mp, i, r + i * kRawBytes, row, hc, nv, &barRaw);
    // a second copy of the gate tensor: block 4 is turned into gate values in place, this one keeps
    // the pre-activations for the derivative of the activation
    if (sigm) seq::fetch_block<T>(mp, 4, r + 6 * kRawBytes, row, hc, nv, &barRaw);
  };
  // start state (16-bit, 8 KB) and end state gradient (fp32, 16 KB) of a chunk into the padded
  // landing zones: three 16-byte asynchronous copies per thread
  auto issue_state = [&](int64_t ci) {   // every thread
    const Item w = split_item(ci, nc, mp.heads);
    const int64_t b = w.bh, c = w.c;
    const T *s0p = (c == 0) ? state + (size_t)b * kDim * kDim : ckpt + ((size_t)b * nc + (c - 1)) * kDim * kDim;
    const float *rp = Rend + (size_t)ci * kDim * kDim;
    cp_async16(sm + oS0L + (tid >> 3) * kS0Ld + (tid & 7) * 16, s0p + (tid >> 3) * kDim + (tid & 7) * 8);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c16 = tid + i * kThreadsB;
      cp_async16(sm + oRL + (c16 >> 4) * kRLd + (c16 & 15) * 16, rp + (c16 >> 4) * kDim + (c16 & 15) * 4);
    }
    cp_async_commit();
  };

  if (tid == 0) {
    umma::mbar_init(&barRaw, 1);
    umma::mbar_init(&barZ, 1);
    umma::mbar_init(&barM, 4);      // TQ1, T7, TQ2, T2: one commit each
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, kTmemCols);
  if (unit_forget) seq::fill_block(raw + kC * kDim, 1.f, tid, kThreadsB);   // constant d-side gate, never loaded
  sync_all();
  dependency_wait();
  const uint32_t tb = __shfl_sync(0xffffffffu, tmem_slot, 0);
  const uint32_t tl = umma::tmem_addr(tb, 32 * q4, 0);
  // Work items of this CTA.  Chunk ci = blockIdx + r * grid for the full rounds r.  The chunks that
  // are left over when the count is not a multiple of the grid would make some CTAs run one whole
  // chunk longer than the others; if there are at most grid / 2 of them, each is split into its two
  // passes (which are independent) over two CTAs instead.
  const int64_t n_full = total / gridDim.x, rem = total - n_full * gridDim.x;
  const bool split_tail = rem > 0 && 2 * rem <= (int64_t)gridDim.x;
  const int64_t n_items =
      n_full + ((split_tail ? (int64_t)blockIdx.x < 2 * rem : (int64_t)blockIdx.x < rem) ? 1 : 0);
  auto item_chunk = [&](int64_t r) -> int64_t {
    return (split_tail && r == n_full) ? n_full * gridDim.x + (blockIdx.x >> 1) : (int64_t)blockIdx.x + r * gridDim.x;
  };
  bool raw_pending = false;      // thread 0
  if (n_items > 0) {
    if (tid == 0) {
      issue_raw(item_chunk(0));
      raw_pending = true;
    }
    issue_state(item_chunk(0));
  }
  const uint32_t aT = umma::smem_u32(sm + oT);
  uint64_t dT[4];      // descriptors of the four tiles
#pragma unroll
  for (int i = 0; i < 4; ++i) dT[i] = desc_sw128(aT + i * kTile);
  uint32_t pz = 0, pm_par = 0;   // mbarrier phase parities

  uint32_t it = 0;
  for (int64_t r = 0; r < n_items; ++r, ++it) {
    const int64_t ci = item_chunk(r);
    const bool half_item = split_tail && r == n_full;
    const int ph_lo = half_item ? (int)(blockIdx.x & 1u) : 0, ph_hi = half_item ? ph_lo + 1 : 2;
    const Item wi = split_item(ci, nc, mp.heads);
    const int64_t b = wi.bh, c = wi.c, t0c = c * kC;
    const int nvalid = (int)((T_ - t0c < kC) ? T_ - t0c : kC);
    // first row and column window of the chunk in the output arrays
    const bool by_row = (mp.flags & seq::kOutByRow) != 0;
    const int64_t row0 = (by_row ? wi.bh : wi.b) * T_ + t0c;
    const int hcol = by_row ? 0 : wi.h * kDim;

    if (!acp::mbar_wait(&barRaw, it & 1u)) s_fail = 1;
    if (tid == 0) raw_pending = false;
    cp_async_wait_all();       // this thread's share of the chunk's start state and end gradient
    __syncthreads();
    if (s_fail) break;
    if (kFused && (sigmoid_gate || q_scale != 1.f)) {      // fused layer: activations applied here
      if (sigmoid_gate) seq::sigmoid_gate_block(raw + 4 * kC * kDim, tid, kThreadsB);
      if (q_scale != 1.f) seq::scale_block(raw + 2 * kC * kDim, q_scale, tid, kThreadsB);
      __syncthreads();
    }
    if (nvalid < kC) {      // partial chunk: identity steps beyond the valid ones
      pad_raw_tail<T>(raw, 6, (1u << 1) | (1u << 4), nvalid, tid, kThreadsB);
      __syncthreads();
    }

#pragma unroll 1
    for (int ph = ph_lo; ph < ph_hi; ++ph) {
      // pass 0: own = k side (other = d side);  pass 1: own = d side
      const int blk_go = ph ? 4 : 1, blk_mo = ph ? 2 : 5, blk_vo = ph ? 3 : 0;   // other: gate, mul, div
      const int blk_gw = ph ? 1 : 4, blk_mw = ph ? 5 : 2, blk_vw = ph ? 0 : 3;   // own
      // What a pass writes before its first barrier - the quarter products and the tiny-gate
      // bookkeeping - the epilogue of the pass before may still be reading: one copy per pass, and no
      // barrier between the passes of an item.
      float *qtot = qtot2 + ph * 8 * kDim;
      float *prd = prd2 + ph * 6 * kDim;
      unsigned long long *fix_mask = fix_mask2 + ph * kDim;
      int &fix_n = fix_n2[ph];

      // ---- stage 1: gate products of the four quarters, then the ratios to the anchor ----
      if (tid == 0) {
        s_bad = 0;
        fix_n = 0;
        fix_rows_n = 0;
      }
      if (tid < kDim) fix_mask[tid] = 0ull;
      float g[16], g_min;
      qtot[(gsw * 4 + tq) * kDim + feat] =
          load_gates16<T>(raw + (gsw ? blk_gw : blk_go) * kC * kDim + feat, tq, g, &g_min);
      __syncthreads();
      if (s_fail) break;      // a wait of the pass before gave up (seen by all after the barrier)
      {
        const float *qt = qtot + gsw * 4 * kDim + feat;
        const float carry = tq == 0 ? qt[kDim] : tq == 3 ? qt[2 * kDim] : 1.f;
        float pm[16];
        if (!ratios16(tq, g, carry, pm)) s_bad = 1;
        if (tq == 1) {
          // Products over the half chunks, once per feature instead of once per use.  Other side:
          // [0] up to the anchor, [1] after it, [2] the whole chunk; own side: [3], [4], [5] = 1 / [3].
          const float up = qt[0] * qt[kDim], after = qt[2 * kDim] * qt[3 * kDim];
          prd[(3 * gsw) * kDim + feat] = up;
          prd[(3 * gsw + 1) * kDim + feat] = after;
          prd[(3 * gsw + 2) * kDim + feat] = gsw ? __fdividef(1.f, up) : up * after;
        }
        if (gsw == 0) {
#pragma unroll
          for (int j = 0; j < 16; ++j) pmo[(16 * tq + j) * kDim + feat] = pm[j];
        } else {
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<float4 *>(pmT + feat * kPmLd + 16 * tq + j) = make_float4(pm[j], pm[j + 1], pm[j + 2], pm[j + 3]);
          if (g_min < kTinyGate)      // rare: some gate of this quarter is tiny
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (fabsf(g[j]) < kTinyGate && 16 * tq + j < nvalid) {   // exact pair sum for this (step, feature) later
              const int slot = atomicAdd(&fix_n, 1);
              if (slot < kFixCap) {
                fix_code[slot] = ((16 * tq + j) << 8) | feat;
                if (atomicOr(&fix_mask[feat], 1ull << (16 * tq + j)) == 0ull) {      // first entry of this feature
                  const int rs = atomicAdd(&fix_rows_n, 1);
                  fix_slot[feat] = rs < kFixRows ? rs : -1;
                  if (rs >= kFixRows) s_bad = 1;
                }
              } else {
                s_bad = 1;
              }
            }
          }
        }
      }
      __syncthreads();

      // ---- stage 2: operands ----
      {   // other side, time-major tiles in shared memory: this thread = four features, steps t and t + 32
        const int f4 = (tid & 15) * 4;
        const float4 o_ref = *reinterpret_cast<const float4 *>(prd + f4);
        const float4 oc_ref = *reinterpret_cast<const float4 *>(prd + kDim + f4);
        const T *r_m = raw + blk_mo * kC * kDim + f4, *r_v = raw + blk_vo * kC * kDim + f4;
        unsigned char *t0p = sm + oT;
#pragma unroll
        for (int i2 = 0; i2 < 2; ++i2) {
          const int t = (tid >> 4) + 32 * i2;
          const float4 pv = *reinterpret_cast<const float4 *>(pmo + t * kDim + f4);
          const float4 m = mul4(Vec4<T>::ld(r_m + t * kDim), pv);
          const float4 v = mul4(Vec4<T>::ld(r_v + t * kDim), rcp4(pv));
          const int o = toff(t, f4);
          *reinterpret_cast<float4 *>(t0p + o) = bias4(m);
          *reinterpret_cast<float4 *>(t0p + kTile + o) = bias4(v);
          *reinterpret_cast<float4 *>(t0p + 2 * kTile + o) = bias4(mul4(m, o_ref));
          *reinterpret_cast<float4 *>(t0p + 3 * kTile + o) = bias4(mul4(v, oc_ref));
        }
      }
      float mw[8], vw[8];      // own-side operand values of this thread, used again by the epilogue
      {   // own side, feature-major A operands in tensor memory: row `own`, steps c0 .. c0 + 7
        const T *r_m = raw + blk_mw * kC * kDim + c0 * kDim + own, *r_v = raw + blk_vw * kC * kDim + c0 * kDim + own;
        const float4 p0 = *reinterpret_cast<const float4 *>(pmT + own * kPmLd + c0);
        const float4 p1 = *reinterpret_cast<const float4 *>(pmT + own * kPmLd + c0 + 4);
        const float pv[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          mw[j] = rna_tf32(Elem<T>::ld(r_m + j * kDim) * pv[j]);
          vw[j] = rna_tf32(Elem<T>::ld(r_v + j * kDim) * __fdividef(1.f, pv[j]));
        }
        tmem_put_dup(tl + cMw, part, h, mw);
        tmem_put_dup(tl + cVw, part, h, vw);
        if (fix_n > 0 && fix_mask[own] != 0ull) {      // rare: the direct pair sums of this feature read its operand rows
          const int rs = fix_slot[own];
          if (rs >= 0) {
            float *row = fix_rows + rs * 2 * kDim + c0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              row[j] = mw[j];
              row[kDim + j] = vw[j];
            }
          }
        }
      }
      // ---- state blocks S2 = W_REF .* S0, R2 = W_63/W_REF .* R as A operands, boundary partial sums ----
      {
        const float w_ref = prd[3 * kDim + own], wc_ref = prd[4 * kDim + own];
        const float4 oc0 = *reinterpret_cast<const float4 *>(prd + 2 * kDim + c0);
        const float4 oc1 = *reinterpret_cast<const float4 *>(prd + 2 * kDim + c0 + 4);
        const float ocv[8] = {oc0.x, oc0.y, oc0.z, oc0.w, oc1.x, oc1.y, oc1.z, oc1.w};
        float sv[8], rv[8];
        if (ph == 0) {        // S(own = k, other = d = c0 + j): a column of the stored blocks
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            sv[j] = Elem<T>::ld(reinterpret_cast<const T *>(sm + oS0L + (c0 + j) * kS0Ld) + own);
            rv[j] = *(reinterpret_cast<const float *>(sm + oRL + (c0 + j) * kRLd) + own);
          }
        } else {              // S(own = d, other = k = c0 + j): a row segment
          const uint4 u = *reinterpret_cast<const uint4 *>(sm + oS0L + own * kS0Ld + c0 * 2);
          const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
          for (int j = 0; j < 8; ++j) sv[j] = Elem<T>::ld(e + j);
          const float4 r0 = *reinterpret_cast<const float4 *>(sm + oRL + own * kRLd + c0 * 4);
          const float4 r1 = *reinterpret_cast<const float4 *>(sm + oRL + own * kRLd + c0 * 4 + 16);
          rv[0] = r0.x; rv[1] = r0.y; rv[2] = r0.z; rv[3] = r0.w;
          rv[4] = r1.x; rv[5] = r1.y; rv[6] = r1.z; rv[7] = r1.w;
        }
        float s2[8], r2[8], acc = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s2[j] = rna_tf32(sv[j] * w_ref);
          r2[j] = rna_tf32(rv[j] * wc_ref);
          acc = fmaf(ocv[j] * s2[j], r2[j], acc);
        }
        tmem_put_dup(tl + cS2, part, h, s2);
        tmem_put_dup(tl + cR2, part, h, r2);
        bndp[cg * kDim + own] = acc;
      }
      umma::tmem_st_wait();
      umma::fence_async_smem();
      sync_all();       // operands complete; in the second pass the raw blocks and the state blocks are consumed

      // ---- first MMA round.  A product is a chain of eight dependent instructions (one per 8
      //      contraction columns, accumulating in place); the tensor core executes instructions in
      //      issue order, so the six independent chains of this round are issued interleaved by ONE
      //      lane and overlap in the pipeline instead of running one after the other. ----
      // Issuing one instruction costs the issuing thread about 30 cycles, so the three products of
      // this round are issued by lanes of three different warps at the same time; each product is
      // two interleaved chains (the two 32-column halves).
      if (warp == 0 || warp == 4 || warp == 8) {
        const uint32_t d0 = tb, d1 = umma::tmem_addr(tb, 16, 0);
        constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
        constexpr uint64_t n1 = (uint64_t)(32 * 128 >> 4);     // B rows 32..63
        if (elect_one()) {
          if (warp == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
              umma::mma_tf32(d0 + cZ, dT[0] + o, dT[1] + o, idesc, ks > 0);                 // Z = Mo_mid Vo_mid^T
              umma::mma_tf32(d1 + cZ, dT[0] + o, dT[1] + n1 + o, idesc, ks > 0);
            }
            umma::mma_commit(&barZ);
          } else if (warp == 4) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
              mma_tf32_ts(d0 + cTQ1, d0 + cS2 + 8 * ks, dT[2] + o, idesc, ks > 0);          // TQ1 = S2 Mo_start^T
              mma_tf32_ts(d1 + cTQ1, d1 + cS2 + 8 * ks, dT[2] + n1 + o, idesc, ks > 0);
            }
            umma::mma_commit(&barM);
          } else {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
              mma_tf32_ts(d0 + cT7, d0 + cR2 + 8 * ks, dT[3] + o, idesc, ks > 0);           // T7 = R2 Vo_end^T
              mma_tf32_ts(d1 + cT7, d1 + cR2 + 8 * ks, dT[3] + n1 + o, idesc, ks > 0);
            }
            umma::mma_commit(&barM);
          }
        }
        __syncwarp();
      }
      if (ph == ph_hi - 1 && r + 1 < n_items) {      // the next item's inputs and state blocks
        if (tid == 0) {
          issue_raw(item_chunk(r + 1));
          raw_pending = true;
        }
        issue_state(item_chunk(r + 1));
      }
      if (tid == 0 && s_bad) atomicExch(rowflag + b, 1);      // the scan kernels redo this batch row

      // ---- Z: mask, round, store as [t][s] (tile 0) and [s][t] (tile 1) ----
      if (!umma::mbar_wait(&barZ, pz)) s_fail = 1;
      pz ^= 1u;
      umma::fence_after_sync();
      {
        const int t = own, s0 = 32 * h + 8 * part;
        float v[8];
        umma::tmem_ld8(tl + cZ + 8 * part, v);
        umma::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (s0 + j <= t) ? bias_tf32(v[j]) : 0.f;
        unsigned char *t0p = sm + oT, *t1p = t0p + kTile;
        *reinterpret_cast<float4 *>(t0p + toff(t, s0)) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(t0p + toff(t, s0 + 4)) = make_float4(v[4], v[5], v[6], v[7]);
#pragma unroll
        for (int j = 0; j < 8; ++j) *reinterpret_cast<float *>(t1p + toff(s0 + j, t)) = v[j];
      }
      umma::fence_async_smem();
      sync_all();
      if (s_fail) break;

      // ---- second MMA round: TQ2 = Vw_mid Z^T, T2 = Mw_mid Z, four interleaved chains ----
      if (warp == 0 || warp == 4) {
        const uint32_t d0 = tb, d1 = umma::tmem_addr(tb, 16, 0);
        constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
        constexpr uint64_t n1 = (uint64_t)(32 * 128 >> 4);
        if (elect_one()) {
          if (warp == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
              mma_tf32_ts(d0 + cTQ2, d0 + cVw + 8 * ks, dT[0] + o, idesc, ks > 0);
              mma_tf32_ts(d1 + cTQ2, d1 + cVw + 8 * ks, dT[0] + n1 + o, idesc, ks > 0);
            }
          } else {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
              mma_tf32_ts(d0 + cT2, d0 + cMw + 8 * ks, dT[1] + o, idesc, ks > 0);
              mma_tf32_ts(d1 + cT2, d1 + cMw + 8 * ks, dT[1] + n1 + o, idesc, ks > 0);
            }
          }
          umma::mma_commit(&barM);
        }
        __syncwarp();
      }
      // ---- tiny gates: pair terms i < t <= s summed directly (runs under the MMAs), one warp per
      //      entry, from the operand rows that the feature's threads left in shared memory ----
      {
        const int n_fix = fix_n < kFixCap ? fix_n : kFixCap;
        const unsigned char *zt = sm + oT;
        // the tile holds Z with the rounding increment but unmasked: the value the tensor core uses
        auto zval = [](const unsigned char *p) {
          return __uint_as_float(*reinterpret_cast<const uint32_t *>(p) & 0xffffe000u);
        };
        // entries go to warps 8 .. 15: warps 0 and 4 are still issuing the second round
        for (int e = warp - 8; e >= 0 && e < n_fix; e += 8) {
          const int code = fix_code[e], t = code >> 8, rs = fix_slot[code & 0xff];
          if (rs < 0) continue;      // no row slot: the batch row is flagged
          const float *row = fix_rows + rs * 2 * kDim;
          // sum_{s >= t} Mw[s] sum_{i < t} Z[s][i] Vw[i]: lanes over i, independent loads over s
          float acc = 0.f;
          for (int i = lane; i < t; i += 32) {
            const unsigned char *zcol = zt + (i >> 5) * kColBlock + ((i & 3) << 2);      // toff(s, i) without the s terms
            const int ic = (i >> 2) & 7;
            float a0 = 0.f, a1 = 0.f;      // two chains: the sums are latency-bound
            int s = t;
            if ((kC - t) & 1) {
              a0 = row[s] * zval(zcol + s * 128 + ((ic ^ (s & 7)) << 4));
              ++s;
            }
#pragma unroll 4
            for (; s < kC; s += 2) {
              a0 = fmaf(row[s], zval(zcol + s * 128 + ((ic ^ (s & 7)) << 4)), a0);
              a1 = fmaf(row[s + 1], zval(zcol + (s + 1) * 128 + ((ic ^ ((s + 1) & 7)) << 4)), a1);
            }
            acc = fmaf(a0 + a1, row[kDim + i], acc);
          }
          acc = warp_sum(acc);
          if (lane == 0) fix_val[e] = acc;
        }
      }
      if (fix_n > 0) __syncthreads();      // the direct sums are visible (fix_n is final since the ratio stage)

      // ---- feature-major epilogue: this thread = row `own`, steps c0 .. c0 + 7 ----
      {
        float pmv[9];
        {
          const float4 p0 = *reinterpret_cast<const float4 *>(pmT + own * kPmLd + c0);
          const float4 p1 = *reinterpret_cast<const float4 *>(pmT + own * kPmLd + c0 + 4);
          pmv[1] = p0.x; pmv[2] = p0.y; pmv[3] = p0.z; pmv[4] = p0.w; pmv[5] = p1.x; pmv[6] = p1.y; pmv[7] = p1.z; pmv[8] = p1.w;
          // ratio of the step before this range; before step 0 it is 1 / W_REF
          pmv[0] = c0 ? pmT[own * kPmLd + c0 - 1] : prd[5 * kDim + own];
        }
        float bnd = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) bnd += bndp[r * kDim + own];
        if (!umma::mbar_wait(&barM, pm_par)) s_fail = 1;
        pm_par ^= 1u;
        umma::fence_after_sync();
        float tq1[8], tq2[8], t2v[8], t7v[8];
        umma::tmem_ld8(tl + cTQ1 + 8 * part, tq1);
        umma::tmem_ld8(tl + cTQ2 + 8 * part, tq2);
        umma::tmem_ld8(tl + cT2 + 8 * part, t2v);
        umma::tmem_ld8(tl + cT7 + 8 * part, t7v);
        umma::tmem_ld_wait();
        float dmu[8], ddv[8], sa[8], sb[8], pre[8], igate[8];      // igate = 1 / gate of the step
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float ip = __fdividef(1.f, pmv[j + 1]);
          dmu[j] = pmv[j + 1] * (tq1[j] + tq2[j]);
          ddv[j] = (t2v[j] + t7v[j]) * ip;
          igate[j] = pmv[j] * ip;
          sa[j] = mw[j] * tq1[j];
          sb[j] = mw[j] * tq2[j] - vw[j] * t2v[j];
          pre[j] = vw[j] * t7v[j];
        }
#pragma unroll
        for (int j = 6; j >= 0; --j) { sa[j] += sa[j + 1]; sb[j] += sb[j + 1]; }   // inclusive suffix sums
        float run = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float v = pre[j]; pre[j] = run; run += v; }   // exclusive prefix
        xc[(0 * 8 + cg) * kDim + own] = sa[0];
        xc[(1 * 8 + cg) * kDim + own] = sb[0];
        xc[(2 * 8 + cg) * kDim + own] = run;
        umma::named_barrier(1 + q4, 128);       // the four warps that share this lane quarter
        float addA = 0.f, addB = 0.f, addP = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float va = xc[(0 * 8 + r) * kDim + own], vb2 = xc[(1 * 8 + r) * kDim + own];
          const float vp = xc[(2 * 8 + r) * kDim + own];
          addA += (r > cg) ? va : 0.f;        // later steps
          addB += (r > cg) ? vb2 : 0.f;
          addP += (r < cg) ? vp : 0.f;        // earlier steps
        }
        const float base_h = addA + addP + bnd;
#pragma unroll
        for (int j = 0; j < 8; ++j) sb[j] += addB;
        if (fix_n > 0) {      // (uniform) tiny gates in this chunk: their pair terms were summed directly
          const int n_fix = fix_n < kFixCap ? fix_n : kFixCap;
          for (int e = 0; e < n_fix; ++e) {
            const int code = fix_code[e], jj = (code >> 8) - c0;
            if ((code & 0xff) == own && (unsigned)jj < 8u) {
              const float v = fix_val[e];
#pragma unroll
              for (int j = 0; j < 8; ++j) sb[j] = (jj == j) ? v : sb[j];
            }
          }
        }
        // 16 consecutive features of one step are 32 contiguous bytes: the results go straight out.
        // Fused layer: the query was scaled on the way in, and the gate tensor holds pre-activations
        // (gate = max(sigmoid(g), 1/8)), so the chain rule is finished here.
        const seq::Out<T> &o_dv = ph ? dx : dk, &o_gt = ph ? df : dfk;
        const bool sig = ph == 0 && sigmoid_gate;
        const T *r_gate = raw + 6 * kC * kDim + c0 * kDim + own;     // pre-activations
        // element pointers of step c0; one row pitch further per step
        T *p_mu = dq.p + (size_t)(row0 + c0) * dq.ld + dq.col + hcol + own;
        T *p_dv = o_dv.p + (size_t)(row0 + c0) * o_dv.ld + o_dv.col + hcol + own;
        T *p_gt = o_gt.p == nullptr ? nullptr : o_gt.p + (size_t)(row0 + c0) * o_gt.ld + o_gt.col + hcol + own;
        // the plain operator and the block-grid form write dense [rows][64] arrays
        const int64_t ld_mu = kFused ? dq.ld : kDim, ld_dv = kFused ? o_dv.ld : kDim, ld_gt = kFused ? o_gt.ld : kDim;
        const float qs = q_scale;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float H = sa[j] + sb[j] + pre[j] + base_h;
          if (c0 + j < nvalid) {
            if (ph == 0) p_mu[j * ld_mu] = (T)(dmu[j] * qs);
            p_dv[j * ld_dv] = (T)ddv[j];
            float dg = H * igate[j];      // H / gate
            if (sig) {      // d gate / d pre-activation, from the pre-activation itself in fp32
              const float e = __expf(-Elem<T>::ld(r_gate + j * kDim));
              const float sg = __fdividef(1.f, 1.f + e);
              dg *= sg > seq::kGateFloor ? sg * sg * e : 0.f;      // s (1 - s) = s^2 e^{-g}
            }
            if (p_gt != nullptr) p_gt[j * ld_gt] = (T)dg;
          }
        }
      }
      umma::fence_before_sync();      // this pass's accumulator reads are ordered before the next barrier
    }
  }
  cp_async_wait_all();
  __syncthreads();      // s_fail of the last pass is visible
  if (tid == 0 && s_fail) {
    atomicExch(status, 1);
    if (raw_pending) acp::mbar_wait(&barRaw, it & 1u);   // bounded: let the copies in flight land
  }
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, kTmemCols);
}

}  // namespace

// mp: tensor maps of x, f, q, k, fk, dO; outs: dx, df, dq, dk, dfk (pointer, row pitch, column) - df may be null.
int lfw_c64_backward_main(const seq::Maps &mp, const void *state, const void *ckpt, const float *Rend,
                          void *const outs[5], const int64_t out_ld[5], const int out_col[5], int *rowflag,
                          int64_t BH, int64_t T_, int dtype, cudaStream_t st) {
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  int n_sm = 0;
  rc = lfw_chunk_sm_count(&n_sm);
  if (rc != T2FW_OK) return rc;
  const int64_t nc = ceil_div64(T_, kC), total = BH * nc;
  const unsigned grid = (unsigned)(total < n_sm ? total : n_sm);
#define T2FW_OUT(TT, i) seq::Out<TT>{(TT *)outs[i], out_ld[i], out_col[i]}
#define T2FW_LAUNCH(TT, FF)                                                                           \
  do {                                                                                                \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_c64_bwd_kernel<TT, FF>,                                  \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemB));       \
    T2FW_CHECK_CUDA(launch_dependent(lfw_c64_bwd_kernel<TT, FF>, dim3(grid), dim3(kThreadsB), kSmemB, st, mp,   \
                                     (const TT *)state, (const TT *)ckpt, Rend, T2FW_OUT(TT, 0), T2FW_OUT(TT, 1), \
                                     T2FW_OUT(TT, 2), T2FW_OUT(TT, 3), T2FW_OUT(TT, 4), rowflag, status, T_, nc,  \
                                     total));                                                         \
  } while (0)
  const bool fused = (mp.flags & (seq::kUnitForget | seq::kSigmoidGate)) != 0 || mp.q_scale != 1.f;
  if (dtype == T2FW_F16) {
    if (fused) T2FW_LAUNCH(__half, true); else T2FW_LAUNCH(__half, false);
  } else {
    if (fused) T2FW_LAUNCH(__nv_bfloat16, true); else T2FW_LAUNCH(__nv_bfloat16, false);
  }
#undef T2FW_LAUNCH
#undef T2FW_OUT
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw

