// C ABI of the library (declared in include/t2fw_b200.h): argument checks and dispatch to the
// kernel launchers.  Nothing here allocates, frees or synchronises.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <initializer_list>

#include "common.cuh"

namespace t2fw {

namespace {
thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};
}  // namespace

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool dependent_launch_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("T2FW_DISABLE_PDL");
    return !(e && e[0] == '1');
  }();
  return on;
}

}  // namespace t2fw

using namespace t2fw;

extern "C" {

const char *t2fw_last_error(void) { return g_err; }

int t2fw_version(void) { return 100; }

int t2fw_device_status(void) {
  const int a = lfw_decode_bulk_status(), b = lfw_chunk_umma_status();
  if (a < 0 || b < 0) return -1;
  return a | b;
}

int64_t t2fw_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int64_t t2fw_lfw_default_ckpt_every(int64_t T, int64_t D, int64_t K, int dtype) {
  (void)T;
  (void)D;
  (void)K;
  (void)dtype;
  return 64;   // the interval the chunked tensor-core kernels are built around
}

int64_t t2fw_lfw_ckpt_slots(int64_t T, int64_t ckpt_every) {
  if (T <= 0 || ckpt_every <= 0) return 0;
  return ceil_div64(T, ckpt_every);
}

static bool decode_bulk_enabled() {
  const char *e = std::getenv("T2FW_DISABLE_DECODE_BULK");
  return !(e && e[0] == '1');
}

static bool chunk_path_enabled() {
  const char *e = std::getenv("T2FW_DISABLE_CHUNK");
  return !(e && e[0] == '1');
}

size_t t2fw_lfw_forward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int dtype,
                                      int64_t ckpt_every) {
  if (T > 1 && chunk_path_enabled() && lfw_chunk_supported(D, K, dtype, ckpt_every))
    return lfw_chunk_forward_scratch_bytes(B, T, ckpt_every);
  if (T > 1 && chunk_path_enabled() && lfw_blocked_supported(D, K, dtype, ckpt_every))
    return lfw_blocked_forward_scratch_bytes(B, T, D, K, ckpt_every);
  return 0;
}

size_t t2fw_lfw_backward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int dtype,
                                       int64_t ckpt_every) {
  if (chunk_path_enabled() && lfw_chunk_supported(D, K, dtype, ckpt_every))
    return lfw_chunk_backward_scratch_bytes(B, T, ckpt_every);
  if (chunk_path_enabled() && lfw_blocked_supported(D, K, dtype, ckpt_every))
    return lfw_blocked_backward_scratch_bytes(B, T, D, K, ckpt_every);
  return 0;
}

static bool dfw_chunk_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("T2FW_DISABLE_DFW_CHUNK");
    return !(e && e[0] == '1');
  }();
  return on;
}

size_t t2fw_dfw_forward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t M, int dtype) {
  if (dfw_chunk_enabled() && dfw_chunk_supported(D, M, dtype)) return dfw_chunk_scratch_bytes(B, T, false);
  return 0;
}

static size_t dfw_scan_backward_scratch(int64_t B, int64_t T, int64_t D, int dtype) {
  // d_value is kept in float next to its 16-bit output for the column pass
  if (dtype == T2FW_F16 || dtype == T2FW_BF16) return align_up((size_t)B * T * D * sizeof(float), 256);
  return 0;
}

size_t t2fw_dfw_backward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t M, int dtype) {
  const size_t scan = dfw_scan_backward_scratch(B, T, D, dtype);
  if (dfw_chunk_enabled() && dfw_chunk_supported(D, M, dtype)) {
    const size_t ch = dfw_chunk_scratch_bytes(B, T, true);
    return ch > scan ? ch : scan;
  }
  return scan;
}

// The tensor-core paths move data in 16-byte units (bulk copies, vector loads and stores).  A
// pointer that is not 16-byte aligned (a view at an odd element offset) takes the scan kernels,
// whose accesses are element-wise.
static bool aligned16(std::initializer_list<const void *> ps) {
  uintptr_t acc = 0;
  for (const void *p : ps) acc |= reinterpret_cast<uintptr_t>(p);
  return (acc & 15u) == 0;
}

static int check_common(int64_t B, int64_t T, int64_t D, int64_t K, int dtype) {
  T2FW_CHECK_ARG(dtype_size(dtype) != 0, "unknown dtype %d", dtype);
  T2FW_CHECK_ARG(B > 0 && T > 0 && D > 0 && K > 0, "sizes must be positive (B=%lld T=%lld D=%lld K=%lld)",
                 (long long)B, (long long)T, (long long)D, (long long)K);
  // one limit for every entry point, so that a forward call never succeeds on a shape whose
  // backward call would be refused
  T2FW_CHECK_ARG(D <= 512 && K <= 512, "state extents up to 512 x 512 are supported (D=%lld, K=%lld)",
                 (long long)D, (long long)K);
  return T2FW_OK;
}

int t2fw_lfw_forward(const void *x, const void *f, const void *q, const void *k,
                     const void *f_key, const void *state, void *outputs, void *ckpt_states,
                     int64_t B, int64_t T, int64_t D, int64_t K, int dtype, int64_t ckpt_every,
                     void *scratch, size_t scratch_bytes, void *stream) {
  int rc = check_common(B, T, D, K, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(x && f && q && k && f_key && state && outputs && ckpt_states, "null pointer argument");
  T2FW_CHECK_ARG(ckpt_every > 0, "ckpt_every must be positive");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (T == 1) {
    const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(f) |
                      reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                      reinterpret_cast<uintptr_t>(f_key) | reinterpret_cast<uintptr_t>(state) |
                      reinterpret_cast<uintptr_t>(outputs) |
                      reinterpret_cast<uintptr_t>(ckpt_states)) & 15u) == 0;
    if (al && decode_bulk_enabled() && lfw_decode_bulk_supported(B, D, K, dtype))
      return lfw_decode_bulk_forward(x, f, q, k, f_key, state, outputs, ckpt_states, B, D, K,
                                     dtype, st);
    if (lfw_decode_supported(D, K, dtype)) {
      rc = lfw_decode_forward(x, f, q, k, f_key, state, outputs, ckpt_states, B, D, K, dtype, st);
      if (rc != T2FW_ERR_UNSUPPORTED) return rc;
    }
  }
  const size_t need = t2fw_lfw_forward_scratch_bytes(B, T, D, K, dtype, ckpt_every);
  if (need != 0 && aligned16({x, f, q, k, f_key, state, outputs, ckpt_states, scratch})) {
    if (scratch == nullptr || scratch_bytes < need) {
      set_error("lfw forward needs %zu bytes of scratch, got %zu", need, scratch_bytes);
      return T2FW_ERR_SCRATCH;
    }
    if (!lfw_chunk_supported(D, K, dtype, ckpt_every))
      return lfw_blocked_forward(x, f, q, k, f_key, state, outputs, ckpt_states, B, T, D, K, dtype,
                                 ckpt_every, scratch, st);
    const int *rowflag = nullptr;
    rc = lfw_chunk_forward(x, f, q, k, f_key, state, outputs, ckpt_states, B, T, dtype, ckpt_every,
                           scratch, st, &rowflag);
    if (rc != T2FW_OK) return rc;
    // batch rows whose gate products left the range the factored form can hold are redone by
    // the scan kernel (it exits at once for all other rows)
    return lfw_scan_forward(x, f, q, k, f_key, state, outputs, ckpt_states, B, T, D, K, dtype,
                            ckpt_every, st, rowflag);
  }
  return lfw_scan_forward(x, f, q, k, f_key, state, outputs, ckpt_states, B, T, D, K, dtype,
                          ckpt_every, st);
}

int t2fw_lfw_backward(const void *grad_output, const void *grad_state, const void *x,
                      const void *f, const void *q, const void *k, const void *f_key,
                      const void *state, const void *ckpt_states, void *d_x, void *d_f, void *d_q,
                      void *d_k, void *d_f_key, void *d_state, int64_t B, int64_t T, int64_t D,
                      int64_t K, int dtype, int64_t ckpt_every, void *scratch,
                      size_t scratch_bytes, void *stream) {
  int rc = check_common(B, T, D, K, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(grad_output && grad_state && x && f && q && k && f_key && state && ckpt_states &&
                     d_x && d_f && d_q && d_k && d_f_key && d_state,
                 "null pointer argument");
  T2FW_CHECK_ARG(ckpt_every > 0, "ckpt_every must be positive");
  const size_t need = t2fw_lfw_backward_scratch_bytes(B, T, D, K, dtype, ckpt_every);
  if (need != 0 && aligned16({grad_output, grad_state, x, f, q, k, f_key, state, ckpt_states, d_x, d_f, d_q,
                              d_k, d_f_key, d_state, scratch})) {
    if (scratch == nullptr || scratch_bytes < need) {
      set_error("lfw backward needs %zu bytes of scratch, got %zu", need, scratch_bytes);
      return T2FW_ERR_SCRATCH;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!lfw_chunk_supported(D, K, dtype, ckpt_every))
      return lfw_blocked_backward(grad_output, grad_state, x, f, q, k, f_key, state, ckpt_states,
                                  d_x, d_f, d_q, d_k, d_f_key, d_state, B, T, D, K, dtype, ckpt_every,
                                  scratch, st);
    const int *rowflag = nullptr;
    rc = lfw_chunk_backward(grad_output, grad_state, x, f, q, k, f_key, state, ckpt_states, d_x,
                            d_f, d_q, d_k, d_f_key, d_state, B, T, dtype, ckpt_every, scratch, st,
                            &rowflag);
    if (rc != T2FW_OK) return rc;
    return lfw_scan_backward(grad_output, grad_state, x, f, q, k, f_key, state, ckpt_states, d_x,
                             d_f, d_q, d_k, d_f_key, d_state, B, T, D, K, dtype, ckpt_every, st,
                             rowflag);
  }
  return lfw_scan_backward(grad_output, grad_state, x, f, q, k, f_key, state, ckpt_states, d_x,
                           d_f, d_q, d_k, d_f_key, d_state, B, T, D, K, dtype, ckpt_every,
                           static_cast<cudaStream_t>(stream));
}

// ---- summary of a sequence segment (time axis split over devices) -------------------------------
size_t t2fw_lfw_segment_summary_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int dtype) {
  if (B <= 0 || T <= 0 || !lfw_chunk_supported(D, K, dtype, 64)) return 0;
  return lfw_segment_summary_scratch_bytes(B, T);
}

int t2fw_lfw_segment_summary(int backward, const void *val_d, const void *gate_d, const void *val_k,
                             const void *gate_k, void *end_state, float *decay_d, float *decay_k, int64_t B,
                             int64_t T, int64_t D, int64_t K, int dtype, void *scratch, size_t scratch_bytes,
                             void *stream) {
  int rc = check_common(B, T, D, K, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(val_d && gate_d && val_k && gate_k && end_state && decay_d && decay_k, "null pointer argument");
  if (!lfw_chunk_supported(D, K, dtype, 64)) {
    set_error("segment summary: D = K = 64 and 16-bit storage only (D=%lld K=%lld dtype %d)", (long long)D, (long long)K,
              dtype);
    return T2FW_ERR_UNSUPPORTED;
  }
  const size_t need = lfw_segment_summary_scratch_bytes(B, T);
  if (scratch == nullptr || scratch_bytes < need) {
    set_error("segment summary needs %zu bytes of scratch, got %zu", need, scratch_bytes);
    return T2FW_ERR_SCRATCH;
  }
  if (!aligned16({val_d, gate_d, val_k, gate_k, end_state, decay_d, decay_k, scratch})) {
    set_error("segment summary: all pointers must be 16-byte aligned");
    return T2FW_ERR_UNSUPPORTED;
  }
  return lfw_segment_summary(backward != 0, val_d, gate_d, val_k, gate_k, end_state, decay_d, decay_k, B, T, dtype,
                             scratch, static_cast<cudaStream_t>(stream));
}

int t2fw_lfw_fold_summaries(int backward, const float *gathered, const float *start, float *at_segment,
                            float *total, int n_segments, int segment, int64_t B, int64_t D, int64_t K,
                            void *stream) {
  T2FW_CHECK_ARG(B > 0 && D > 0 && K > 0, "sizes must be positive (B=%lld D=%lld K=%lld)", (long long)B, (long long)D,
                 (long long)K);
  T2FW_CHECK_ARG(n_segments > 0 && segment >= 0 && segment < n_segments, "segment %d of %d", segment, n_segments);
  T2FW_CHECK_ARG(gathered && start && at_segment, "null pointer argument");
  T2FW_CHECK_ARG(B <= (int64_t)1 << 40 && D <= 4096 && K <= 4096, "sizes out of range");
  return lfw_fold_summaries(backward != 0, gathered, start, at_segment, total, n_segments, segment, B, D, K,
                            static_cast<cudaStream_t>(stream));
}

// ---- fused decay-rule layer (heads read in place from the projection output) -------------------
static int check_fused(int64_t B, int64_t T, int64_t H, int dtype) {
  T2FW_CHECK_ARG(B > 0 && T > 0 && H > 0, "sizes must be positive (B=%lld T=%lld H=%lld)", (long long)B,
                 (long long)T, (long long)H);
  if (dtype != T2FW_F16 && dtype != T2FW_BF16) {
    set_error("fused layer: 16-bit storage only (dtype %d)", dtype);
    return T2FW_ERR_UNSUPPORTED;
  }
  return T2FW_OK;
}

size_t t2fw_lfw_fused_scratch_bytes(int64_t B, int64_t T, int64_t H, int dtype) {
  if (B <= 0 || T <= 0 || H <= 0 || (dtype != T2FW_F16 && dtype != T2FW_BF16)) return 0;
  return lfw_fused_scratch_bytes(B, T, (int)H);
}

int t2fw_lfw_fused_forward(const void *qkvg, const void *state, void *outputs, void *ckpt_states, int64_t B,
                           int64_t T, int64_t H, int dtype, void *scratch, size_t scratch_bytes, void *stream) {
  int rc = check_fused(B, T, H, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(qkvg && state && outputs && ckpt_states, "null pointer argument");
  const size_t need = lfw_fused_scratch_bytes(B, T, (int)H);
  if (scratch == nullptr || scratch_bytes < need) {
    set_error("lfw fused forward needs %zu bytes of scratch, got %zu", need, scratch_bytes);
    return T2FW_ERR_SCRATCH;
  }
  if (!aligned16({qkvg, state, outputs, ckpt_states, scratch})) {
    set_error("lfw fused forward: all pointers must be 16-byte aligned");
    return T2FW_ERR_UNSUPPORTED;
  }
  return lfw_fused_forward(qkvg, state, outputs, ckpt_states, B, T, (int)H, dtype, scratch,
                           static_cast<cudaStream_t>(stream));
}

int t2fw_lfw_fused_backward(const void *grad_output, const void *grad_state, const void *qkvg, const void *state,
                            const void *ckpt_states, void *d_qkvg, void *d_state, int64_t B, int64_t T, int64_t H,
                            int dtype, void *scratch, size_t scratch_bytes, void *stream) {
  int rc = check_fused(B, T, H, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(grad_output && grad_state && qkvg && state && ckpt_states && d_qkvg && d_state,
                 "null pointer argument");
  const size_t need = lfw_fused_scratch_bytes(B, T, (int)H);
  if (scratch == nullptr || scratch_bytes < need) {
    set_error("lfw fused backward needs %zu bytes of scratch, got %zu", need, scratch_bytes);
    return T2FW_ERR_SCRATCH;
  }
  if (!aligned16({grad_output, grad_state, qkvg, state, ckpt_states, d_qkvg, d_state, scratch})) {
    set_error("lfw fused backward: all pointers must be 16-byte aligned");
    return T2FW_ERR_UNSUPPORTED;
  }
  return lfw_fused_backward(grad_output, grad_state, qkvg, state, ckpt_states, d_qkvg, d_state, B, T, (int)H, dtype,
                            scratch, static_cast<cudaStream_t>(stream));
}

int t2fw_dfw_forward(const void *q, const void *k, const void *v, const void *state,
                     void *outputs, void *final_state, void *delta, int64_t B, int64_t T,
                     int64_t D, int64_t M, int dtype, void *stream) {
  int rc = check_common(B, T, D, M, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(q && k && v && state && outputs && final_state && delta, "null pointer argument");
  return dfw_scan_forward(q, k, v, state, outputs, final_state, delta, B, T, D, M, dtype,
                          static_cast<cudaStream_t>(stream));
}

int t2fw_dfw_forward_ws(const void *q, const void *k, const void *v, const void *state,
                        void *outputs, void *final_state, void *delta, int64_t B, int64_t T,
                        int64_t D, int64_t M, int dtype, void *scratch, size_t scratch_bytes,
                        void *stream) {
  int rc = check_common(B, T, D, M, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(q && k && v && state && outputs && final_state && delta, "null pointer argument");
  const size_t need = t2fw_dfw_forward_scratch_bytes(B, T, D, M, dtype);
  if (need != 0 && aligned16({q, k, v, state, outputs, final_state, delta, scratch})) {
    if (scratch == nullptr || scratch_bytes < need) {
      set_error("dfw forward needs %zu bytes of scratch, got %zu", need, scratch_bytes);
      return T2FW_ERR_SCRATCH;
    }
    return dfw_chunk_forward(q, k, v, state, outputs, final_state, delta, B, T, dtype, scratch,
                             static_cast<cudaStream_t>(stream));
  }
  return dfw_scan_forward(q, k, v, state, outputs, final_state, delta, B, T, D, M, dtype,
                          static_cast<cudaStream_t>(stream));
}

int t2fw_dfw_backward(const void *grad_output, const void *grad_state, const void *q,
                      const void *k, const void *delta, const void *final_state, void *d_q,
                      void *d_k, void *d_v, void *d_state, int64_t B, int64_t T, int64_t D,
                      int64_t M, int dtype, void *scratch, size_t scratch_bytes, void *stream) {
  int rc = check_common(B, T, D, M, dtype);
  if (rc != T2FW_OK) return rc;
  T2FW_CHECK_ARG(grad_output && grad_state && q && k && delta && final_state && d_q && d_k &&
                     d_v && d_state,
                 "null pointer argument");
  const size_t need = t2fw_dfw_backward_scratch_bytes(B, T, D, M, dtype);
  void *dv_acc = d_v;  // float / double outputs double as the accumulation-type copy
  if (need != 0) {
    if (scratch == nullptr || scratch_bytes < need) {
      set_error("dfw backward needs %zu bytes of scratch, got %zu", need, scratch_bytes);
      return T2FW_ERR_SCRATCH;
    }
    dv_acc = scratch;
  }
  if (dfw_chunk_enabled() && dfw_chunk_supported(D, M, dtype) &&
      aligned16({grad_output, grad_state, q, k, delta, final_state, d_q, d_k, d_v, d_state, scratch}))
    return dfw_chunk_backward(grad_output, grad_state, q, k, delta, final_state, d_q, d_k, d_v, d_state,
                              B, T, dtype, scratch, static_cast<cudaStream_t>(stream));
  return dfw_scan_backward(grad_output, grad_state, q, k, delta, final_state, d_q, d_k, d_v,
                           d_state, dv_acc, B, T, D, M, dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
