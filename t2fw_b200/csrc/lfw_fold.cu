// Combining the segment summaries of a sequence whose TIME axis is split over devices (decay rule).
// A segment acts on the state as  S_end = (A G^T) .* S_start + L  (t2fw_lfw_segment_summary), so the
// state that enters segment r is the fold of segments 0 .. r-1 over the state before step 0, and the
// state gradient that enters segment r from behind is the fold of segments n-1 .. r+1 over the
// gradient of the final state.  One launch does the whole fold: a thread owns one state element and
// walks the segments in order, so the result does not depend on the number of launches or on the
// order in which summaries arrived.  The recurrence restated is t2fw/torch.py:21-28 of the
// reference, which has no multi-device code.
#include "common.cuh"

namespace t2fw {

namespace {

// gathered: [n][B][D*K + D + K] fp32 = per segment (L [D][K], A [D], G [K]) of every batch row.
// forward:  S = start; for j = 0 .. n-1: (j == r: at_r = S);  S = A_j G_j^T .* S + L_j;   total = S
// backward: R = start; for j = n-1 .. r+1: R = A_j G_j^T .* R + L_j;                       at_r = R
template <bool kBackward>
__global__ void __launch_bounds__(256)
lfw_fold_kernel(const float *__restrict__ gathered, const float *__restrict__ start, float *__restrict__ at_r,
                float *__restrict__ total, int n, int r, int64_t B, int D, int K) {
  const int64_t per = (int64_t)D * K, rec = per + D + K;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * per) return;
  const int64_t b = i / per, e = i - b * per;
  const int d = (int)(e / K), k = (int)(e - (int64_t)d * K);
  float s = start[i];
  if (!kBackward) {
    for (int j = 0; j < n; ++j) {
      const float *p = gathered + ((int64_t)j * B + b) * rec;
      if (j == r) at_r[i] = s;
      s = p[per + d] * p[per + D + k] * s + p[e];
    }
    if (total != nullptr) total[i] = s;
  } else {
    for (int j = n - 1; j > r; --j) {
      const float *p = gathered + ((int64_t)j * B + b) * rec;
      s = p[per + d] * p[per + D + k] * s + p[e];
    }
    at_r[i] = s;
  }
}

}  // namespace

int lfw_fold_summaries(bool backward, const float *gathered, const float *start, float *at_rank, float *total,
                       int n, int r, int64_t B, int64_t D, int64_t K, cudaStream_t st) {
  const int64_t elems = B * D * K;
  const unsigned grid = (unsigned)ceil_div64(elems, 256);
  if (backward)
    lfw_fold_kernel<true><<<grid, 256, 0, st>>>(gathered, start, at_rank, total, n, r, B, (int)D, (int)K);
  else
    lfw_fold_kernel<false><<<grid, 256, 0, st>>>(gathered, start, at_rank, total, n, r, B, (int)D, (int)K);
  T2FW_CHECK_LAUNCH(1);
  return T2FW_OK;
}

}  // namespace t2fw
