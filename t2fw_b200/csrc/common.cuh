// Shared helpers for the sm_100a kernels: element-type traits, warp reductions, error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/t2fw_b200.h"

namespace t2fw {

// ---- error plumbing -------------------------------------------------------------------
void set_error(const char *fmt, ...);
void count_launch(int n = 1);

#define T2FW_CHECK_ARG(cond, ...)                 \
  do {                                            \
    if (!(cond)) {                                \
      ::t2fw::set_error(__VA_ARGS__);             \
      return T2FW_ERR_BAD_ARG;                    \
    }                                             \
  } while (0)

#define T2FW_CHECK_CUDA(expr)                                                        \
  do {                                                                               \
    cudaError_t _e = (expr);                                                         \
    if (_e != cudaSuccess) {                                                         \
      ::t2fw::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),      \
                        __FILE__, __LINE__);                                         \
      return T2FW_ERR_CUDA;                                                          \
    }                                                                                \
  } while (0)

#define T2FW_CHECK_LAUNCH(n)                                                         \
  do {                                                                               \
    ::t2fw::count_launch(n);                                                         \
    T2FW_CHECK_CUDA(cudaGetLastError());                                             \
  } while (0)

// ---- programmatic dependent launch -------------------------------------------------------
// A kernel launched with launch_dependent() may be scheduled while the kernel before it in the
// stream is still running: its prologue (barrier initialisation, tensor-memory allocation) and its
// launch latency then overlap that kernel's tail.  dependency_wait() blocks until the earlier
// kernel has completed and its writes are visible; every such kernel calls it before its first
// access to global memory (so completion is transitive along the stream), then lets the next
// kernel in.  T2FW_DISABLE_PDL=1 turns the launch attribute off (the device calls are then no-ops).
#ifdef __CUDACC__
__device__ __forceinline__ void dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif
bool dependent_launch_enabled();      // api.cu
template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- element types ----------------------------------------------------------------------
// Acc<T> is the type the recurrences are carried in: float for 16/32-bit storage, double for
// double.  (The reference accumulates in the storage type, t2fw/csrc/lfw_kernel.cu:49.)
template <typename T> struct Elem;
template <> struct Elem<__half> {
  using acc = float;
  static __device__ __forceinline__ float ld(const __half *p) { return __half2float(*p); }
  static __device__ __forceinline__ void st(__half *p, float v) { *p = __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  using acc = float;
  static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Elem<float> {
  using acc = float;
  static __device__ __forceinline__ float ld(const float *p) { return *p; }
  static __device__ __forceinline__ void st(float *p, float v) { *p = v; }
};
template <> struct Elem<double> {
  using acc = double;
  static __device__ __forceinline__ double ld(const double *p) { return *p; }
  static __device__ __forceinline__ void st(double *p, double v) { *p = v; }
};

template <typename A>
__device__ __forceinline__ A warp_sum(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case T2FW_F16: case T2FW_BF16: return 2;
    case T2FW_F32: return 4;
    case T2FW_F64: return 8;
    default: return 0;
  }
}

// Launchers implemented in the kernel translation units.  All return a T2FW_* status.
int lfw_scan_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                     const void *state, void *out, void *ckpt, int64_t B, int64_t T, int64_t D,
                     int64_t K, int dtype, int64_t C, cudaStream_t st,
                     const int *rowflag = nullptr);
int lfw_scan_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                      const void *k, const void *fk, const void *state, const void *ckpt,
                      void *dx, void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B,
                      int64_t T, int64_t D, int64_t K, int dtype, int64_t C, cudaStream_t st,
                      const int *rowflag = nullptr);
// chunked tensor-core path (D = K = 64, 16-bit storage, checkpoint interval a multiple of 64)
bool lfw_chunk_supported(int64_t D, int64_t K, int dtype, int64_t ckpt_every);
size_t lfw_chunk_forward_scratch_bytes(int64_t B, int64_t T, int64_t ckpt_every);
int lfw_chunk_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                      const void *state, void *out, void *ckpt, int64_t B, int64_t T, int dtype,
                      int64_t ckpt_every, void *scratch, cudaStream_t st, const int **rowflag_out);
size_t lfw_chunk_backward_scratch_bytes(int64_t B, int64_t T, int64_t ckpt_every);
int lfw_chunk_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                       const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
                       void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B, int64_t T,
                       int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st,
                       const int **rowflag_out);
// the same for a batch of D x K states cut into (D/64) x (K/64) blocks: sequence inputs dense
// [B*T][D] / [B*T][K] read in place; states, checkpoints and all results per block
// ([B * nd * nk][..][64][64] and [B * nd * nk][T][64], block (i, j) of item b at b * nd * nk + i * nk + j)
int lfw_chunk_forward_grid(const void *x, const void *f, const void *q, const void *k, const void *fk,
                           const void *state_blocks, void *out_blocks, void *ckpt_blocks, int64_t B, int64_t T,
                           int nd, int nk, int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st,
                           const int **rowflag_out);
int lfw_chunk_backward_grid(const void *go, const void *gs_blocks, const void *x, const void *f, const void *q,
                            const void *k, const void *fk, const void *state_blocks, const void *ckpt_blocks,
                            void *dx, void *df, void *dq, void *dk, void *dfk, void *ds_blocks, int64_t B, int64_t T,
                            int nd, int nk, int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st,
                            const int **rowflag_out);
// state shapes that are grids of 64 x 64 blocks (D, K multiples of 64, up to 256)
bool lfw_blocked_supported(int64_t D, int64_t K, int dtype, int64_t ckpt_every);
size_t lfw_blocked_forward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int64_t ckpt_every);
size_t lfw_blocked_backward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int64_t ckpt_every);
int lfw_blocked_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                        const void *state, void *out, void *ckpt, int64_t B, int64_t T, int64_t D,
                        int64_t K, int dtype, int64_t ckpt_every, void *scratch, cudaStream_t st);
int lfw_blocked_backward(const void *go, const void *gs, const void *x, const void *f, const void *q,
                         const void *k, const void *fk, const void *state, const void *ckpt, void *dx,
                         void *df, void *dq, void *dk, void *dfk, void *ds, int64_t B, int64_t T,
                         int64_t D, int64_t K, int dtype, int64_t ckpt_every, void *scratch,
                         cudaStream_t st);
// what a sequence segment does to the state / state gradient (D = K = 64, 16-bit): see lfw_c64_host.cu
size_t lfw_segment_summary_scratch_bytes(int64_t B, int64_t T);
int lfw_segment_summary(bool backward, const void *val_d, const void *gate_d, const void *val_k, const void *gate_k,
                        void *end_state, float *A_out, float *G_out, int64_t B, int64_t T, int dtype, void *scratch,
                        cudaStream_t st);
// fold of gathered segment summaries into the state / state gradient that enters segment r (lfw_fold.cu)
int lfw_fold_summaries(bool backward, const float *gathered, const float *start, float *at_rank, float *total,
                       int n, int r, int64_t B, int64_t D, int64_t K, cudaStream_t st);
// fused layer form of the chunked path: qkvg [B][T][4*H*64] read in place (lfw_c64_host.cu)
size_t lfw_fused_scratch_bytes(int64_t B, int64_t T, int H);
int lfw_fused_forward(const void *qkvg, const void *state, void *out, void *ckpt, int64_t B, int64_t T, int H,
                      int dtype, void *scratch, cudaStream_t st);
int lfw_fused_backward(const void *go, const void *gs, const void *qkvg, const void *state, const void *ckpt,
                       void *d_qkvg, void *ds, int64_t B, int64_t T, int H, int dtype, void *scratch,
                       cudaStream_t st);
int lfw_chunk_umma_status();
bool lfw_decode_bulk_supported(int64_t B, int64_t D, int64_t K, int dtype);
int lfw_decode_bulk_forward(const void *x, const void *f, const void *q, const void *k,
                            const void *fk, const void *state, void *out, void *new_state,
                            int64_t B, int64_t D, int64_t K, int dtype, cudaStream_t st);
int lfw_decode_bulk_status();
bool lfw_decode_supported(int64_t D, int64_t K, int dtype);
int lfw_decode_forward(const void *x, const void *f, const void *q, const void *k, const void *fk,
                       const void *state, void *out, void *new_state, int64_t B, int64_t D,
                       int64_t K, int dtype, cudaStream_t st);
// chunked delta rule (dfw_chunk.cu): D = M = 64, 16-bit storage
bool dfw_chunk_supported(int64_t D, int64_t M, int dtype);
size_t dfw_chunk_scratch_bytes(int64_t B, int64_t T, bool backward);
int dfw_chunk_forward(const void *q, const void *k, const void *v, const void *state, void *out,
                      void *final_state, void *delta, int64_t B, int64_t T, int dtype, void *scratch,
                      cudaStream_t st);
int dfw_chunk_backward(const void *go, const void *gs, const void *q, const void *k, const void *delta,
                       const void *final_state, void *dq, void *dk, void *dv, void *ds, int64_t B, int64_t T,
                       int dtype, void *scratch, cudaStream_t st);
int dfw_scan_forward(const void *q, const void *k, const void *v, const void *state, void *out,
                     void *fin, void *delta, int64_t B, int64_t T, int64_t D, int64_t M, int dtype,
                     cudaStream_t st);
int dfw_scan_backward(const void *go, const void *gs, const void *q, const void *k,
                      const void *delta, const void *fin, void *dq, void *dk, void *dv, void *ds,
                      void *dv_acc, int64_t B, int64_t T, int64_t D, int64_t M, int dtype,
                      cudaStream_t st);

}  // namespace t2fw
