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
EncodeFn g_encode = nullptr;
std::once_flag g_once;
cudaError_t g_lookup_error = cudaSuccess;
}  // namespace

int make_map(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t ld) {
  std::call_once(g_once, [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    g_lookup_error = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (g_lookup_error == cudaSuccess && qres == cudaDriverEntryPointSuccess) g_encode = reinterpret_cast<EncodeFn>(fn);
  });
  if (g_encode == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver (%s)", cudaGetErrorString(g_lookup_error));
    return T2FW_ERR_CUDA;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld * 2) % 16 != 0 || cols % 8 != 0) {
    set_error("tensor map: base, row pitch and width must be multiples of 16 bytes");
    return T2FW_ERR_UNSUPPORTED;
  }
  // The driver call needs the device's context current on THIS host thread; a thread that has only
  // used the runtime lazily (autograd's backward worker) may not have it bound yet.
  T2FW_CHECK_CUDA(cudaFree(nullptr));
  const cuuint64_t dims[2] = {cols, rows};               // innermost first
  const cuuint64_t strides[1] = {ld * 2};                // bytes between rows
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (rows=%llu cols=%llu ld=%llu)", (int)rc,
              (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
    return T2FW_ERR_CUDA;
  }
  return T2FW_OK;
}

}  // namespace seq
}  // namespace t2fw
