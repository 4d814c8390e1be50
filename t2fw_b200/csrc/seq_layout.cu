// Host side of seq_layout.cuh: tensor maps through the driver entry point (the library does not
// link against libcuda; the runtime hands out the function).
#include <mutex>

#include <cudaTypedefs.h>

#include "seq_layout.cuh"

namespace t2fw {
namespace seq {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
using RetainFn = CUresult (*)(CUcontext *, CUdevice);
using ReleaseFn = CUresult (*)(CUdevice);
using SetCurrentFn = CUresult (*)(CUcontext);
EncodeFn g_encode = nullptr;
RetainFn g_retain = nullptr;
ReleaseFn g_release = nullptr;
SetCurrentFn g_set_current = nullptr;
std::once_flag g_once;
cudaError_t g_lookup_error = cudaSuccess;

void *entry_point(const char *name) {
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  const cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess) g_lookup_error = e;
  return (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) ? fn : nullptr;
}

// Makes the current device's primary context current on this host thread with driver calls only
// (they are allowed while a stream of the thread is being captured, unlike a runtime call that
// would do the same as a side effect).  The runtime holds its own reference to the context, so
// the one taken here is given back at once.
bool bind_primary_context() {
  if (!g_retain || !g_release || !g_set_current) return false;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  CUcontext ctx = nullptr;
  if (g_retain(&ctx, (CUdevice)dev) != CUDA_SUCCESS) return false;
  const bool ok = g_set_current(ctx) == CUDA_SUCCESS;
  g_release((CUdevice)dev);
  return ok;
}
}  // namespace

int make_map(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t ld) {
  std::call_once(g_once, [] {
    g_encode = reinterpret_cast<EncodeFn>(entry_point("cuTensorMapEncodeTiled"));
    g_retain = reinterpret_cast<RetainFn>(entry_point("cuDevicePrimaryCtxRetain"));
    g_release = reinterpret_cast<ReleaseFn>(entry_point("cuDevicePrimaryCtxRelease"));
    g_set_current = reinterpret_cast<SetCurrentFn>(entry_point("cuCtxSetCurrent"));
  });
  if (g_encode == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver (%s)", cudaGetErrorString(g_lookup_error));
    return T2FW_ERR_CUDA;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld * 2) % 16 != 0 || cols % 8 != 0) {
    set_error("tensor map: base, row pitch and width must be multiples of 16 bytes");
    return T2FW_ERR_UNSUPPORTED;
  }
  const cuuint64_t dims[2] = {cols, rows};               // innermost first
  const cuuint64_t strides[1] = {ld * 2};                // bytes between rows
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t estr[2] = {1, 1};
  auto encode = [&] {
    return g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult rc = encode();
  // The driver call needs the device's context current on THIS host thread; a thread that has only
  // used the runtime lazily (autograd's backward worker) may not have it bound yet.
  if ((rc == CUDA_ERROR_INVALID_CONTEXT || rc == CUDA_ERROR_NOT_INITIALIZED) && bind_primary_context()) rc = encode();
  if (rc != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (rows=%llu cols=%llu ld=%llu)", (int)rc,
              (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
    return T2FW_ERR_CUDA;
  }
  return T2FW_OK;
}

}  // namespace seq
}  // namespace t2fw
