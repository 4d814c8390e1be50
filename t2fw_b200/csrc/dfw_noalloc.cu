// Delta-rule backward for hosts that cannot allocate device memory.
//
// t2fw_dfw_backward needs, for 16-bit element types, a float copy of d_value ([B,T,D]) that
// the row pass writes and the column pass reads; normally the caller allocates it.  Some
// callers cannot: a serving runtime that reserved the whole GPU for its own pool at start-up
// (so a later cudaMalloc fails), a latency-critical loop that must not hit cudaMalloc's
// implicit device synchronisation, or a foreign-function bridge that can pass an operator's
// inputs and outputs but has no way to hand over extra buffers.  For them the scratch lives
// in a fixed array inside the library image.  The price: every GPU that loads the library
// holds these 16 MiB until the process exits, the problem size is capped, and all calls on
// a device share the one array.
#include <mutex>

#include "common.cuh"

namespace {

// Capacity in floats: B*T*D of a 16-bit problem must not exceed this (16 MiB).
constexpr size_t kMaxElems = size_t(4) << 20;

static __device__ __align__(256) float g_dv_scratch[kMaxElems];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float *g_scratch_addr[kMaxDevices] = {};

// In host code `g_dv_scratch` is only a handle; the address the kernels can use has to be
// asked for, once per device, while that device is current.
int scratch_for_current_device(float **out) {
  int dev = -1;
  T2FW_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    t2fw::set_error("dfw backward (no-alloc): device index %d out of range", dev);
    return T2FW_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void *p = nullptr;
    T2FW_CHECK_CUDA(cudaGetSymbolAddress(&p, g_dv_scratch));
    g_scratch_addr[dev] = static_cast<float *>(p);
  }
  *out = g_scratch_addr[dev];
  return T2FW_OK;
}

}  // namespace

extern "C" {

size_t t2fw_dfw_backward_noalloc_max_elems(void) { return kMaxElems; }

int t2fw_dfw_backward_noalloc(const void *grad_output, const void *grad_state, const void *q,
                              const void *k, const void *delta, const void *final_state,
                              void *d_q, void *d_k, void *d_v, void *d_state, int64_t B,
                              int64_t T, int64_t D, int64_t M, int dtype, void *stream) {
  T2FW_CHECK_ARG(t2fw::dtype_size(dtype) != 0, "unknown dtype %d", dtype);
  T2FW_CHECK_ARG(B > 0 && T > 0 && D > 0 && M > 0,
                 "sizes must be positive (B=%lld T=%lld D=%lld M=%lld)", (long long)B,
                 (long long)T, (long long)D, (long long)M);
  T2FW_CHECK_ARG(grad_output && grad_state && q && k && delta && final_state && d_q && d_k &&
                     d_v && d_state,
                 "null pointer argument");
  void *dv_acc = d_v;  // float / double outputs are their own accumulation-type copy
  if (dtype == T2FW_F16 || dtype == T2FW_BF16) {
    // each factor is bounded first, so that the product below cannot wrap around
    const bool fits = (unsigned long long)B <= kMaxElems && (unsigned long long)T <= kMaxElems &&
                      (unsigned long long)D <= kMaxElems &&
                      (unsigned long long)B * (unsigned long long)T <= kMaxElems;
    const unsigned long long need = fits ? (unsigned long long)B * T * D : ~0ull;
    if (need > kMaxElems) {
      t2fw::set_error(
          "dfw backward (no-alloc): B*T*D = %llu exceeds the built-in scratch of %zu elements; "
          "use t2fw_dfw_backward with caller-provided scratch",
          need, kMaxElems);
      return T2FW_ERR_SCRATCH;
    }
    float *p = nullptr;
    const int rc = scratch_for_current_device(&p);
    if (rc != T2FW_OK) return rc;
    dv_acc = p;  // fully rewritten by the row pass before the column pass reads it
  }
  return t2fw::dfw_scan_backward(grad_output, grad_state, q, k, delta, final_state, d_q, d_k, d_v,
                                 d_state, dv_acc, B, T, D, M, dtype,
                                 static_cast<cudaStream_t>(stream));
}

}  // extern "C"
