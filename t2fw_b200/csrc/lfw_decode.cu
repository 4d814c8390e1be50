// Decay-rule decode step (T = 1): S' = (f fk^T) .* S + x k^T, o = S' q for B independent states.
//
// This is the reference's forward (t2fw/csrc/lfw_kernel.cu:18-59 plus the einsum of
// t2fw/csrc/lfw.cpp:45) at seqlen 1, the shape its benchmark measures
// (tests/benchmark.py:104-105).  It is pure streaming: each state element is read once and
// written once, so the kernel is built around 128-bit loads and stores of 8 storage elements
// along K, fp32 arithmetic in registers, and a shuffle reduction over the K/8 threads that
// share a row for o = S' q.  Several rows per thread keep independent 16-byte loads in flight.
#include "common.cuh"

namespace t2fw {

namespace {

template <typename T> struct Pack8;
template <> struct Pack8<__half> {
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
template <> struct Pack8<__nv_bfloat16> {
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

constexpr int kDecodeThreads = 128;
constexpr int kRowsInFlight = 4;

// One CTA per batch element.  Thread (rr, kc) handles the 8 columns kc*8.. of rows
// rr, rr+RP, rr+2RP, ...  where RP = threads / (K/8).
template <typename T>
__global__ void __launch_bounds__(kDecodeThreads)
lfw_decode_kernel(const T *__restrict__ x, const T *__restrict__ f, const T *__restrict__ q,
                  const T *__restrict__ k, const T *__restrict__ fk, const T *__restrict__ state,
                  T *__restrict__ out, T *__restrict__ new_state, int D, int K) {
  const int64_t b = blockIdx.x;
  const int KT = K >> 3;
  const int kc = threadIdx.x % KT;
  const int rr = threadIdx.x / KT;
  const int RP = kDecodeThreads / KT;

  float g[8], kk[8], qq[8];
  Pack8<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(fk + b * K) + kc), g);
  Pack8<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(k + b * K) + kc), kk);
  Pack8<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(q + b * K) + kc), qq);

  const uint4 *sin = reinterpret_cast<const uint4 *>(state + b * (int64_t)D * K);
  uint4 *sout = reinterpret_cast<uint4 *>(new_state + b * (int64_t)D * K);

  for (int base = 0; base < D; base += RP * kRowsInFlight) {
    uint4 raw[kRowsInFlight];
    float xs[kRowsInFlight], as[kRowsInFlight];
#pragma unroll
    for (int i = 0; i < kRowsInFlight; ++i) {
      const int row = base + rr + i * RP;
      const bool in = row < D;
      raw[i] = in ? __ldcs(sin + (int64_t)row * KT + kc) : make_uint4(0, 0, 0, 0);
      xs[i] = in ? Elem<T>::ld(x + b * D + row) : 0.f;
      as[i] = in ? Elem<T>::ld(f + b * D + row) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < kRowsInFlight; ++i) {
      const int row = base + rr + i * RP;
      const bool in = row < D;
      float s[8];
      Pack8<T>::unpack(raw[i], s);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        s[e] = s[e] * (as[i] * g[e]) + xs[i] * kk[e];
        acc += s[e] * qq[e];
      }
      if (in) __stcs(sout + (int64_t)row * KT + kc, Pack8<T>::pack(s));
      for (int o = KT >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (in && kc == 0) Elem<T>::st(out + b * D + row, acc);
    }
  }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

bool lfw_decode_supported(int64_t D, int64_t K, int dtype) {
  if (dtype != T2FW_F16 && dtype != T2FW_BF16) return false;
  if (K < 8 || K > 256 || (K & (K - 1)) != 0) return false;  // K/8 threads share a row
  return D >= 1 && D <= 65536;
}

int lfw_decode_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                       const void *state, void *out, void *new_state, int64_t B, int64_t D,
                       int64_t K, int dtype, cudaStream_t st) {
  if (!lfw_decode_supported(D, K, dtype) || !aligned16(q) || !aligned16(k) || !aligned16(fk) ||
      !aligned16(state) || !aligned16(new_state)) {
    set_error("lfw decode: unsupported shape or unaligned pointers");
    return T2FW_ERR_UNSUPPORTED;
  }
  if (dtype == T2FW_F16)
    lfw_decode_kernel<__half><<<(unsigned)B, kDecodeThreads, 0, st>>>(
        (const __half *)x, (const __half *)f, (const __half *)q, (const __half *)k,
        (const __half *)fk, (const __half *)state, (__half *)out, (__half *)new_state, (int)D,
        (int)K);
  else
    lfw_decode_kernel<__nv_bfloat16><<<(unsigned)B, kDecodeThreads, 0, st>>>(
        (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)f, (const __nv_bfloat16 *)q,
        (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)fk, (const __nv_bfloat16 *)state,
        (__nv_bfloat16 *)out, (__nv_bfloat16 *)new_state, (int)D, (int)K);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw
