// Decay-rule decode step (T = 1) as a persistent, bulk-async-copy pipelined streaming kernel.
//
// Same arithmetic as lfw_decode.cu (the reference's forward at seqlen 1,
// t2fw/csrc/lfw_kernel.cu:18-59 + t2fw/csrc/lfw.cpp:45).  The D x K state of one batch row
// (8 KB at D = K = 64 in fp16) and its five input vectors are brought into shared memory by
// the copy engine (cp.async.bulk global -> shared, completion counted on an mbarrier), updated
// in place with fp32 arithmetic, and streamed back with cp.async.bulk shared -> global.  Each
// CTA walks batch rows b = blockIdx.x, blockIdx.x + gridDim.x, ... with a ring of kStages
// buffers, so several rows per SM are in flight without holding them in registers.
//
// Every wait on an mbarrier is bounded: if it does not complete within kSpinLimit polls the CTA
// records the failure in *status and leaves after draining its own outstanding copies.
#include "common.cuh"

namespace t2fw {

namespace {

constexpr int kThreads = 128;
constexpr int kStages = 3;
constexpr uint32_t kSpinLimit = 1u << 19;   // polls (each may suspend up to ~2 us) before giving up

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
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
  return ok != 0;
}
// bounded wait; returns false on timeout
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *dst, const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(smem_u32(src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <typename T> struct Cvt8;
template <> struct Cvt8<__half> {
  static __device__ __forceinline__ void unpack(const uint4 &u, float (&v)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(h[i]);
      v[2 * i] = p.x;
      v[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
    uint4 u;
    __half2 *h = reinterpret_cast<__half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    return u;
  }
};
template <> struct Cvt8<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(const uint4 &u, float (&v)[8]) {
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __bfloat1622float2(h[i]);
      v[2 * i] = p.x;
      v[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return u;
  }
};

// Stage layout (bytes): state [D*K*2] | fk [K*2] | k [K*2] | q [K*2] | x [D*2] | f [D*2] | out [D*2]
template <typename T>
__global__ void __launch_bounds__(kThreads)
lfw_decode_bulk_kernel(const T *__restrict__ x, const T *__restrict__ f, const T *__restrict__ q,
                       const T *__restrict__ k, const T *__restrict__ fk, const T *__restrict__ state,
                       T *__restrict__ out, T *__restrict__ new_state, int B, int D, int K,
                       int stage_bytes, int *__restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ int s_fail;
  const int KT = K >> 3;
  const int kc = threadIdx.x % KT;
  const int rr = threadIdx.x / KT;
  const int RP = kThreads / KT;
  const uint32_t sbytes = (uint32_t)D * K * sizeof(T), kbytes = (uint32_t)K * sizeof(T),
                 dbytes = (uint32_t)D * sizeof(T);
  const uint32_t tx = sbytes + 3 * kbytes + 2 * dbytes;
  const int n_items = (B - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue_load = [&](int item) {
    const int64_t b = (int64_t)blockIdx.x + (int64_t)item * gridDim.x;
    unsigned char *st = smem + (size_t)(item % kStages) * stage_bytes;
    uint64_t *bar = &full[item % kStages];
    mbar_expect_tx(bar, tx);
    bulk_g2s(st, state + b * (int64_t)D * K, sbytes, bar);
    bulk_g2s(st + sbytes, fk + b * K, kbytes, bar);
    bulk_g2s(st + sbytes + kbytes, k + b * K, kbytes, bar);
    bulk_g2s(st + sbytes + 2 * kbytes, q + b * K, kbytes, bar);
    bulk_g2s(st + sbytes + 3 * kbytes, x + b * D, dbytes, bar);
    bulk_g2s(st + sbytes + 3 * kbytes + dbytes, f + b * D, dbytes, bar);
  };

  if (threadIdx.x == 0)
    for (int i = 0; i < kStages - 1 && i < n_items; ++i) issue_load(i);

  for (int item = 0; item < n_items; ++item) {
    const int s = item % kStages;
    const uint32_t parity = (uint32_t)(item / kStages) & 1u;
    if (!mbar_wait(&full[s], parity)) s_fail = 1;   // benign race: every writer stores 1
    __syncthreads();
    if (s_fail) break;

    unsigned char *st = smem + (size_t)s * stage_bytes;
    uint4 *sst = reinterpret_cast<uint4 *>(st);
    const T *sfk = reinterpret_cast<const T *>(st + sbytes);
    const T *sk = reinterpret_cast<const T *>(st + sbytes + kbytes);
    const T *sq = reinterpret_cast<const T *>(st + sbytes + 2 * kbytes);
    const T *sx = reinterpret_cast<const T *>(st + sbytes + 3 * kbytes);
    const T *sf = reinterpret_cast<const T *>(st + sbytes + 3 * kbytes + dbytes);
    T *so = reinterpret_cast<T *>(st + sbytes + 3 * kbytes + 2 * dbytes);

    float g[8], kk[8], qq[8];
    Cvt8<T>::unpack(reinterpret_cast<const uint4 *>(sfk)[kc], g);
    Cvt8<T>::unpack(reinterpret_cast<const uint4 *>(sk)[kc], kk);
    Cvt8<T>::unpack(reinterpret_cast<const uint4 *>(sq)[kc], qq);
    for (int base = 0; base < D; base += RP) {
      const int row = base + rr;
      const bool in = row < D;
      float sv[8];
      Cvt8<T>::unpack(in ? sst[row * KT + kc] : make_uint4(0, 0, 0, 0), sv);
      const float xs = in ? Elem<T>::ld(sx + row) : 0.f, as = in ? Elem<T>::ld(sf + row) : 0.f;
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sv[e] = sv[e] * (as * g[e]) + xs * kk[e];
        acc += sv[e] * qq[e];
      }
      if (in) sst[row * KT + kc] = Cvt8<T>::pack(sv);
      for (int o = KT >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (in && kc == 0) Elem<T>::st(so + row, acc);
    }
    fence_async_smem();      // make the generic-proxy writes visible to the copy engine
    __syncthreads();
    if (threadIdx.x == 0) {
      const int64_t b = (int64_t)blockIdx.x + (int64_t)item * gridDim.x;
      bulk_s2g(new_state + b * (int64_t)D * K, st, sbytes);
      bulk_s2g(out + b * D, so, dbytes);
      bulk_commit();
      const int nxt = item + kStages - 1;
      if (nxt < n_items) {
        // the buffer being refilled was stored from one iteration ago: allow only the newest
        // store group to be still reading shared memory
        bulk_wait_read<1>();
        issue_load(nxt);
      }
    }
  }
  if (threadIdx.x == 0) {
    bulk_wait_all();
    if (s_fail) atomicExch(status, 1);
  }
}

}  // namespace

// The decode call takes no scratch, so a kernel that gave up waiting reports through this
// module-scope word; the host can read it with lfw_decode_bulk_status().
__device__ int g_decode_status = 0;

namespace {
constexpr int kMaxDev = 64;
int g_sms[kMaxDev] = {};
int *g_status_addr[kMaxDev] = {};
bool g_attr_set[kMaxDev][2] = {};
}  // namespace

bool lfw_decode_bulk_supported(int64_t B, int64_t D, int64_t K, int dtype) {
  if (dtype != T2FW_F16 && dtype != T2FW_BF16) return false;
  if (K < 8 || K > 256 || (K & (K - 1)) != 0) return false;
  if (D < 8 || (D % 8) != 0) return false;
  const size_t stage = align_up((size_t)D * K * 2 + 3 * K * 2 + 3 * D * 2, 128);
  return stage * kStages <= 200 * 1024 && B >= 1 && B < (1ll << 31);
}

int lfw_decode_bulk_forward(const void *x, const void *f, const void *q, const void *k,
                            const void *fk, const void *state, void *out, void *new_state,
                            int64_t B, int64_t D, int64_t K, int dtype, cudaStream_t st) {
  const int stage = (int)align_up((size_t)D * K * 2 + 3 * K * 2 + 3 * D * 2, 128);
  const size_t smem = (size_t)stage * kStages;
  int dev = 0;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDev) {
    set_error("lfw decode: device index %d out of range", dev);
    return T2FW_ERR_UNSUPPORTED;
  }
  if (g_status_addr[dev] == nullptr) {   // first call on this device (do it outside stream capture)
    T2FW_CHECK_CUDA(cudaDeviceGetAttribute(&g_sms[dev], cudaDevAttrMultiProcessorCount, dev));
    void *p = nullptr;
    T2FW_CHECK_CUDA(cudaGetSymbolAddress(&p, g_decode_status));
    g_status_addr[dev] = static_cast<int *>(p);
  }
  const int sms = g_sms[dev];
  int *status = g_status_addr[dev];
  const int per_sm = (int)((220 * 1024) / (smem + 1024));
  int64_t grid = (int64_t)sms * (per_sm < 1 ? 1 : per_sm);
  if (grid > B) grid = B;
  const int ti = dtype == T2FW_F16 ? 0 : 1;
  if (!g_attr_set[dev][ti]) {
    if (ti == 0)
      T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_decode_bulk_kernel<__half>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    else
      T2FW_CHECK_CUDA(cudaFuncSetAttribute(lfw_decode_bulk_kernel<__nv_bfloat16>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    g_attr_set[dev][ti] = true;
  }
  if (dtype == T2FW_F16) {
    lfw_decode_bulk_kernel<__half><<<(unsigned)grid, kThreads, smem, st>>>(
        (const __half *)x, (const __half *)f, (const __half *)q, (const __half *)k,
        (const __half *)fk, (const __half *)state, (__half *)out, (__half *)new_state, (int)B,
        (int)D, (int)K, stage, status);
  } else {
    lfw_decode_bulk_kernel<__nv_bfloat16><<<(unsigned)grid, kThreads, smem, st>>>(
        (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)f, (const __nv_bfloat16 *)q,
        (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)fk, (const __nv_bfloat16 *)state,
        (__nv_bfloat16 *)out, (__nv_bfloat16 *)new_state, (int)B, (int)D, (int)K, stage, status);
  }
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

// Non-zero if a decode kernel ever gave up waiting for its copies (synchronises the device).
int lfw_decode_bulk_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace t2fw
