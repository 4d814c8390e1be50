// Outputs of the chunked decay-rule forward on the tcgen05 tensor core (D = K = 64, 16-bit
// storage, chunks of 64 steps): the third phase after the chunk-local states and the carry over
// chunks.  Replaces the reference's materialised states and output einsum
// (t2fw/csrc/lfw_kernel.cu:43-57, t2fw/csrc/lfw.cpp:45).
//
// Per chunk, with S0 the state at the chunk start (the caller's state or the 16-bit checkpoint the
// carry wrote; notation of lfw_c64.cuh):
//     P   = tril( (q pm_g) (k / pm_g)^T )                       in-chunk decays, k side
//     O^  = (q G_t) (A_REF .* S0)^T  +  P (x / pm_a)            [t][d]
//     o_t = pm_a[t] .* O^_t
// i.e. three 64 x 64 x 64 contractions, all on TF32 operand tiles in shared memory with fp32
// accumulators in tensor memory.
//
// One persistent CTA of 16 warps per SM.  The five raw 8 KB input blocks of a chunk arrive by bulk
// asynchronous copies into one of two buffers (the next chunk is fetched while this one is
// computed); thread (gate side, 16-step quarter, feature) walks its steps with a running gate
// product (stage 1: ratio tables), then the operand tiles are written element-wise with 16-byte
// stores (stage 2); one elected lane issues the MMAs; the accumulators come
// back time-major (a thread owns one step and eight features), so the 16-bit outputs leave as
// 16-byte stores.
#include <type_traits>

#include "lfw_c64.cuh"
#include "seq_layout.cuh"

namespace t2fw {

using namespace c64;

int lfw_chunk_status_ptr(int **out);   // lfw_c64_local.cu
int lfw_chunk_sm_count(int *out);

namespace {

constexpr int kThreadsF = 512;
constexpr int kPmLd = 68;                          // row stride (floats) of the padded ratio tables
// shared-memory map (bytes from the 1024-byte aligned base)
constexpr int oT = 0;                              // tiles: 0 Qmid -> P, 1 Kmid, 2 Qstart, 3 Xmid (feature-major), 4 S0'
constexpr int oPmk = oT + 5 * kTile;               // pm_g[t][k]
constexpr int oPmF = oPmk + kC * kDim * 4;         // pm_a[d][t]
constexpr int oPmA = oPmF + kDim * kPmLd * 4;      // pm_a[t][d]
constexpr int oQt = oPmA + kC * kPmLd * 4;         // quarter products [2 sides][4][64]
constexpr int kS0Ld = 144;                         // row stride (bytes) of the start-state landing zone
constexpr int oS0L = oQt + 2 * 4 * kDim * 4;       // start state of a chunk, [64][kS0Ld] 16-bit
constexpr int oRaw = oS0L + kDim * kS0Ld;           // [2 buffers] x, f, q, k, fk
constexpr int kSmemF = oRaw + 2 * 5 * kRawBytes + 1024;   // + slack for the 1024-byte alignment
static_assert(oRaw % 128 == 0 && oS0L % 16 == 0, "copy destination alignment");
static_assert(kSmemF + 256 <= 227 * 1024, "shared memory limit");

constexpr int cP = 0, cO = 32;                     // tensor-memory columns

template <typename T>
__global__ void __launch_bounds__(kThreadsF, 1)
lfw_c64_fwd_kernel(const __grid_constant__ seq::Maps mp, const T *__restrict__ state, const T *__restrict__ ckpt,
                   const seq::Out<T> out, int *__restrict__ rowflag, int *__restrict__ status, int64_t T_,
                   int64_t nc, int64_t total) {
  extern __shared__ __align__(1024) unsigned char sm_raw[];
  unsigned char *sm = sm_raw + ((1024u - (umma::smem_u32(sm_raw) & 1023u)) & 1023u);   // swizzle atoms are 1024-byte aligned
  __shared__ __align__(8) uint64_t barRaw[2], barP, barO;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_fail, s_bad;

  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  // stage 1: gate side (0: k side, 1: d side), quarter of the chunk, feature
  const int gs = warp >> 3, tq = (warp >> 1) & 3, feat = (warp & 1) * 32 + lane;
  // accumulator read-out: lane quarter, column part, column half (lane set), row in the quarter
  const int q4 = warp & 3, part = warp >> 2, h = lane >> 4, fl = lane & 15;
  // state tile: row d, eight columns
  const int sr = tid & 63, sc0 = (tid >> 6) * 8;

  float *pmk = reinterpret_cast<float *>(sm + oPmk);
  float *pmF = reinterpret_cast<float *>(sm + oPmF);
  float *pmA = reinterpret_cast<float *>(sm + oPmA);
  float *qtot = reinterpret_cast<float *>(sm + oQt);

  // tensors: 0 x, 1 f, 2 q, 3 k, 4 fk
  const bool unit_forget = (mp.flags & seq::kUnitForget) != 0;
  auto issue_raw = [&](int64_t ci, int buf) {     // thread 0 only: one copy per tensor
    const Item w = split_item(ci, nc, mp.heads);
    const int row = (int)(w.b * T_ + w.c * kC), hc = w.h;
    const int nv = (int)((T_ - (int64_t)w.c * kC < kC) ? T_ - (int64_t)w.c * kC : kC);
    unsigned char *r = sm + oRaw + buf * 5 * kRawBytes;
    const uint32_t per = (mp.flags & seq::kContiguous) ? (uint32_t)nv * kDim * sizeof(T) : (uint32_t)kRawBytes;
    acp::mbar_expect_tx(&barRaw[buf], (unit_forget ? 4u : 5u) * per);
#pragma unroll
    for (int i = 0; i < 5; ++i)
      if (!(i == 1 && unit_forget)) seq::fetch_block<T>(mp, i, r + i * kRawBytes, row, hc, nv, &barRaw[buf]);
  };

  // start state of a chunk (the caller's state for the first chunk of a row, else the checkpoint
  // written by the carry): one 16-byte asynchronous copy per thread into the padded landing zone
  auto issue_state = [&](int64_t ci) {   // every thread
    const Item w = split_item(ci, nc, mp.heads);
    const int64_t b = w.bh, c = w.c;
    const T *s0p = (c == 0) ? state + (size_t)b * kDim * kDim : ckpt + ((size_t)b * nc + (c - 1)) * kDim * kDim;
    cp_async16(sm + oS0L + (tid >> 3) * kS0Ld + (tid & 7) * 16, s0p + (tid >> 3) * kDim + (tid & 7) * 8);
    cp_async_commit();
  };

  if (tid == 0) {
    umma::mbar_init(&barRaw[0], 1);
    umma::mbar_init(&barRaw[1], 1);
    umma::mbar_init(&barP, 1);
    umma::mbar_init(&barO, 1);
    umma::mbar_fence_init();
    s_fail = 0;
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 64);
  if (unit_forget) {      // the d-side gate block of both buffers is the constant 1 and never loaded
    seq::fill_block(reinterpret_cast<T *>(sm + oRaw + kRawBytes), 1.f, tid, kThreadsF);
    seq::fill_block(reinterpret_cast<T *>(sm + oRaw + 6 * kRawBytes), 1.f, tid, kThreadsF);
  }
  sync_all();
  dependency_wait();
  const uint32_t tb = __shfl_sync(0xffffffffu, tmem_slot, 0);
  const uint32_t tl = umma::tmem_addr(tb, 32 * q4, 0);
  uint32_t n_issued[2] = {0u, 0u}, n_landed[2] = {0u, 0u};      // thread 0: bulk-copy rounds per buffer
  if ((int64_t)blockIdx.x < total) {
    if (tid == 0) {
      issue_raw(blockIdx.x, 0);
      ++n_issued[0];
    }
    issue_state(blockIdx.x);
  }
  const uint32_t aT = umma::smem_u32(sm + oT);
  const uint64_t dT0 = desc_sw128(aT), dT1 = desc_sw128(aT + kTile), dT2 = desc_sw128(aT + 2 * kTile);
  const uint64_t dT3 = desc_sw128(aT + 3 * kTile), dT4 = desc_sw128(aT + 4 * kTile);

  uint32_t it = 0;
  for (int64_t ci = blockIdx.x; ci < total; ci += gridDim.x, ++it) {
    const int buf = it & 1;
    const Item wi = split_item(ci, nc, mp.heads);
    const int64_t b = wi.bh, c = wi.c, t0c = c * kC;      // b: problem row (batch item x head)
    const int nvalid = (int)((T_ - t0c < kC) ? T_ - t0c : kC);
    T *raw = reinterpret_cast<T *>(sm + oRaw + buf * 5 * kRawBytes);
    const bool by_row = (mp.flags & seq::kOutByRow) != 0;
    T *orow = out.p + ((by_row ? wi.bh : wi.b) * T_ + t0c) * out.ld + out.col + (by_row ? 0 : wi.h * kDim);

    if (tid == 0) {
      s_bad = 0;
      if (ci + gridDim.x < total) {      // the other buffer was released at the end of the previous chunk
        issue_raw(ci + gridDim.x, buf ^ 1);
        ++n_issued[buf ^ 1];
      }
    }
    cp_async_wait_all();       // this thread's share of this chunk's start state (requested one chunk ahead)
    if (acp::mbar_wait(&barRaw[buf], (it >> 1) & 1u)) {
      if (tid == 0) ++n_landed[buf];
    } else {
      s_fail = 1;
    }
    __syncthreads();
    if (s_fail) break;
    if ((mp.flags & seq::kSigmoidGate) || mp.q_scale != 1.f) {      // fused layer: activations applied here
      if (mp.flags & seq::kSigmoidGate) seq::sigmoid_gate_block(raw + 4 * kC * kDim, tid, kThreadsF);
      if (mp.q_scale != 1.f) seq::scale_block(raw + 2 * kC * kDim, mp.q_scale, tid, kThreadsF);
      __syncthreads();
    }
    if (nvalid < kC) {      // partial chunk: identity steps beyond the valid ones
      pad_raw_tail<T>(raw, 5, (1u << 1) | (1u << 4), nvalid, tid, kThreadsF);
      __syncthreads();
    }

    // ---- stage 1: gate products of the four quarters, then the ratios to the anchor ----
    float g[16];
    qtot[(gs * 4 + tq) * kDim + feat] = load_gates16<T>(raw + (gs ? 1 : 4) * kC * kDim + feat, tq, g);
    __syncthreads();
    {
      const float *qt = qtot + gs * 4 * kDim + feat;
      const float carry = tq == 0 ? qt[kDim] : tq == 3 ? qt[2 * kDim] : 1.f;
      float pm[16];
      if (!ratios16(tq, g, carry, pm)) s_bad = 1;
      if (gs == 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) pmk[(16 * tq + j) * kDim + feat] = pm[j];
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) pmA[(16 * tq + j) * kPmLd + feat] = pm[j];
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4 *>(pmF + feat * kPmLd + 16 * tq + j) = make_float4(pm[j], pm[j + 1], pm[j + 2], pm[j + 3]);
      }
    }
    __syncthreads();

    // ---- stage 2: operand tiles ----
    {   // k side, time-major: this thread = four features, steps t and t + 32
      const int f4 = (tid & 15) * 4;
      const float4 g_ref = mul4(*reinterpret_cast<const float4 *>(qtot + f4),
                                *reinterpret_cast<const float4 *>(qtot + kDim + f4));
      const T *r_q = raw + 2 * kC * kDim + f4, *r_k = raw + 3 * kC * kDim + f4;
      unsigned char *t0p = sm + oT;
#pragma unroll
      for (int i2 = 0; i2 < 2; ++i2) {
        const int t = (tid >> 4) + 32 * i2;
        const float4 pv = *reinterpret_cast<const float4 *>(pmk + t * kDim + f4);
        const float4 qm = mul4(Vec4<T>::ld(r_q + t * kDim), pv);
        const float4 km = mul4(Vec4<T>::ld(r_k + t * kDim), rcp4(pv));
        const int o = toff(t, f4);
        *reinterpret_cast<float4 *>(t0p + o) = bias4(qm);
        *reinterpret_cast<float4 *>(t0p + kTile + o) = bias4(km);
        *reinterpret_cast<float4 *>(t0p + 2 * kTile + o) = bias4(mul4(qm, g_ref));
      }
    }
    {   // d side, feature-major: this thread = features 2 * lane, 2 * lane + 1, steps 4 * warp .. + 3
      const int f0 = 2 * lane, t = 4 * warp;
      const T *r_x = raw + t * kDim + f0;
      float2 x2[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) x2[j] = Vec2<T>::ld(r_x + j * kDim);
      const float4 i0 = rcp4(*reinterpret_cast<const float4 *>(pmF + f0 * kPmLd + t));
      const float4 i1 = rcp4(*reinterpret_cast<const float4 *>(pmF + (f0 + 1) * kPmLd + t));
      unsigned char *tX = sm + oT + 3 * kTile;
      *reinterpret_cast<float4 *>(tX + toff(f0, t)) = bias4(mul4(make_float4(x2[0].x, x2[1].x, x2[2].x, x2[3].x), i0));
      *reinterpret_cast<float4 *>(tX + toff(f0 + 1, t)) = bias4(mul4(make_float4(x2[0].y, x2[1].y, x2[2].y, x2[3].y), i1));
    }
    // ---- state tile S0' = A_REF .* S0 ----
    {
      const float a_ref = qtot[4 * kDim + sr] * qtot[5 * kDim + sr];
      const uint4 u = *reinterpret_cast<const uint4 *>(sm + oS0L + sr * kS0Ld + sc0 * 2);
      const T *e = reinterpret_cast<const T *>(&u);
      const float4 s_lo = make_float4(Elem<T>::ld(e), Elem<T>::ld(e + 1), Elem<T>::ld(e + 2), Elem<T>::ld(e + 3));
      const float4 s_hi = make_float4(Elem<T>::ld(e + 4), Elem<T>::ld(e + 5), Elem<T>::ld(e + 6), Elem<T>::ld(e + 7));
      unsigned char *tS = sm + oT + 4 * kTile;
      *reinterpret_cast<float4 *>(tS + toff(sr, sc0)) =
          make_float4(bias_tf32(s_lo.x * a_ref), bias_tf32(s_lo.y * a_ref), bias_tf32(s_lo.z * a_ref),
                      bias_tf32(s_lo.w * a_ref));
      *reinterpret_cast<float4 *>(tS + toff(sr, sc0 + 4)) =
          make_float4(bias_tf32(s_hi.x * a_ref), bias_tf32(s_hi.y * a_ref), bias_tf32(s_hi.z * a_ref),
                      bias_tf32(s_hi.w * a_ref));
    }
    umma::fence_async_smem();
    sync_all();       // tiles complete, raw buffer and start state consumed
    if (ci + gridDim.x < total) issue_state(ci + gridDim.x);

    // A product is a chain of eight dependent instructions; the tensor core executes in issue
    // order, so one lane issues the independent chains interleaved and they overlap in the pipeline.
    if (warp == 0) {
      const uint32_t d0 = tb, d1 = umma::tmem_addr(tb, 16, 0);
      constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
      constexpr uint64_t n1 = (uint64_t)(32 * 128 >> 4);     // B rows 32..63
      if (elect_one()) {
        // P first and on its own barrier: the state term runs while P is masked and stored
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
          umma::mma_tf32(d0 + cP, dT0 + o, dT1 + o, idesc, ks > 0);             // P = Qmid Kmid^T
          umma::mma_tf32(d1 + cP, dT0 + o, dT1 + n1 + o, idesc, ks > 0);
        }
        umma::mma_commit(&barP);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
          umma::mma_tf32(d0 + cO, dT2 + o, dT4 + o, idesc, ks > 0);             // O^ = Qstart S0'^T
          umma::mma_tf32(d1 + cO, dT2 + o, dT4 + n1 + o, idesc, ks > 0);
        }
      }
      __syncwarp();
      if (tid == 0 && s_bad) atomicExch(rowflag + b, 1);      // the scan kernel redoes this batch row
    }
    // ---- P: mask, round, store as the [t][s] operand (over Qmid, which only the P product reads) ----
    if (!umma::mbar_wait(&barP, it & 1u)) s_fail = 1;
    umma::fence_after_sync();
    {
      const int t = 16 * q4 + fl, s0 = 32 * h + 8 * part;
      float v[8];
      umma::tmem_ld8(tl + cP + 8 * part, v);
      umma::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (s0 + j <= t) ? bias_tf32(v[j]) : 0.f;
      unsigned char *tP = sm + oT;
      *reinterpret_cast<float4 *>(tP + toff(t, s0)) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4 *>(tP + toff(t, s0 + 4)) = make_float4(v[4], v[5], v[6], v[7]);
    }
    umma::fence_async_smem();
    sync_all();
    if (s_fail) break;
    if (warp == 0) {     // the same lane as above: O^ += P Xmid follows O^ = ... in issue order
      const uint32_t d0 = tb, d1 = umma::tmem_addr(tb, 16, 0);
      constexpr uint32_t idesc = umma::make_idesc_tf32(64, 32, false, false);
      constexpr uint64_t n1 = (uint64_t)(32 * 128 >> 4);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t o = (uint64_t)(((ks >> 2) * kColBlock + (ks & 3) * 32) >> 4);
          umma::mma_tf32(d0 + cO, dT0 + o, dT3 + o, idesc, true);
          umma::mma_tf32(d1 + cO, dT0 + o, dT3 + n1 + o, idesc, true);
        }
        umma::mma_commit(&barO);
      }
      __syncwarp();
    }
    {
      const int t = 16 * q4 + fl, d0 = 32 * h + 8 * part;
      const float4 p0 = *reinterpret_cast<const float4 *>(pmA + t * kPmLd + d0);
      const float4 p1 = *reinterpret_cast<const float4 *>(pmA + t * kPmLd + d0 + 4);
      if (!umma::mbar_wait(&barO, it & 1u)) s_fail = 1;
      umma::fence_after_sync();
      float v[8];
      umma::tmem_ld8(tl + cO + 8 * part, v);
      umma::tmem_ld_wait();
      if (t < nvalid) {
        __align__(16) T o[8];
        o[0] = (T)(v[0] * p0.x); o[1] = (T)(v[1] * p0.y); o[2] = (T)(v[2] * p0.z); o[3] = (T)(v[3] * p0.w);
        o[4] = (T)(v[4] * p1.x); o[5] = (T)(v[5] * p1.y); o[6] = (T)(v[6] * p1.z); o[7] = (T)(v[7] * p1.w);
        *reinterpret_cast<uint4 *>(orow + (size_t)t * out.ld + d0) = *reinterpret_cast<const uint4 *>(o);
      }
    }
    // No barrier here: the next chunk writes nothing before the barrier at its start (which every
    // thread reaches only after this read-out), and that barrier also spreads s_fail.
    umma::fence_before_sync();
  }
  cp_async_wait_all();
  __syncthreads();      // s_fail of the last chunk is visible
  if (tid == 0) {
    if (s_fail) atomicExch(status, 1);
    // bounded: let copies that are still in flight land before the CTA leaves
    for (int bb = 0; bb < 2; ++bb)
      if (n_issued[bb] > n_landed[bb]) acp::mbar_wait(&barRaw[bb], n_landed[bb] & 1u);
  }
  sync_all();
  if (warp == 0) umma::tmem_dealloc(tb, 64);
}

}  // namespace

// mp: tensor maps of x, f, q, k, fk; state / ckpt [BH][.][64][64]; the outputs go to out.
int lfw_c64_forward_out(const seq::Maps &mp, const void *state, const void *ckpt, void *out, int64_t out_ld,
                        int out_col, int *rowflag, int64_t BH, int64_t T_, int dtype, cudaStream_t st) {
  int *status = nullptr;
  int rc = lfw_chunk_status_ptr(&status);
  if (rc != T2FW_OK) return rc;
  int n_sm = 0;
  rc = lfw_chunk_sm_count(&n_sm);
  if (rc != T2FW_OK) return rc;
  const int64_t nc = ceil_div64(T_, kC), total = BH * nc;
  const unsigned grid = (unsigned)(total < n_sm ? total : n_sm);
#define T2FW_LAUNCH(TT)                                                                              \
  do {                                                                                               \
    T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_c64_fwd_kernel<TT>,                                     \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemF));      \
    T2FW_CHECK_CUDA(launch_dependent(lfw_c64_fwd_kernel<TT>, dim3(grid), dim3(kThreadsF), kSmemF, st, mp,       \
                                     (const TT *)state, (const TT *)ckpt, seq::Out<TT>{(TT *)out, out_ld, out_col}, \
                                     rowflag, status, T_, nc, total));                               \
  } while (0)
  if (dtype == T2FW_F16) T2FW_LAUNCH(__half); else T2FW_LAUNCH(__nv_bfloat16);
#undef T2FW_LAUNCH
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw
