/*
 * t2fw_b200 — C ABI of the B200 (sm_100a) fast-weight recurrence library.
 *
 * This is the seam a host binding links against: plain pointers, 64-bit sizes, an opaque
 * stream handle (a cudaStream_t passed as void*), an integer status.  No torch types.
 * All data pointers are DEVICE pointers to dense row-major arrays; every entry point is
 * asynchronous on the given stream and never synchronises, allocates or frees.
 * Inputs are never written.
 *
 * Shapes (the reference's names):
 *   value/forget/outputs and their gradients ... [B, T, D]
 *   query/key/f_key and their gradients ........ [B, T, K]   (K is "M" in the delta rule)
 *   state, next_state and their gradients ...... [B, D, K]
 *   ckpt_states ................................ [B, n_slots, D, K], slot j = state after step
 *                                                min((j+1)*ckpt_every, T); the last slot is S_T
 *
 * Limits: D <= 512 and K <= 512 in every entry point (T2FW_ERR_BAD_ARG otherwise; forward and
 * backward share the limit, so a training step never fails only at its backward call).
 * Alignment: any element-aligned pointer is accepted; the tensor-core paths need all pointers
 * (scratch included) 16-byte aligned and the library takes its element-wise scan kernels, which
 * are much slower, when one is not.
 *
 * Each function below names the reference interface it replaces (path inside the reference
 * project : lines).
 */
#ifndef T2FW_B200_H
#define T2FW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types; the reference dispatches half, float and double
 * (t2fw/csrc/lfw_kernel.cu:157, AT_DISPATCH_FLOATING_TYPES_AND_HALF); bf16 is an addition */
enum {
  T2FW_F16 = 0,
  T2FW_BF16 = 1,
  T2FW_F32 = 2,
  T2FW_F64 = 3
};

/* status codes (0 = success) */
enum {
  T2FW_OK = 0,
  T2FW_ERR_BAD_ARG = 1,     /* null pointer, non-positive size, unknown dtype ... */
  T2FW_ERR_UNSUPPORTED = 2, /* shape outside what the kernels cover */
  T2FW_ERR_SCRATCH = 3,     /* scratch buffer missing or too small */
  T2FW_ERR_CUDA = 4         /* a CUDA runtime call or launch failed */
};

/* Text of the last error raised on the calling thread ("" if none). */
const char *t2fw_last_error(void);

/* Library version (major*10000 + minor*100 + patch). */
int t2fw_version(void);

/* Number of kernel launches this process has issued through the library so far. */
int64_t t2fw_launch_count(void);

/* 0 if no kernel of the library has ever given up a bounded wait on this device (the kernels
 * never spin forever: a wait that does not complete sets a flag and the kernel returns), a
 * positive value if one has, negative if the flag could not be read.  Synchronises the device. */
int t2fw_device_status(void);

/* Checkpoint interval the library recommends for a problem, and the slot count that follows
 * from an interval.  The reference stores the state of EVERY step
 * (t2fw/csrc/lfw_kernel.cu:140-144); here only every ckpt_every-th state is kept and the
 * backward pass recomputes the rest.  Any positive interval is accepted; multiples of 64 run on
 * the tensor-core kernels (for D, K multiples of 64 and 16-bit storage), other intervals on the
 * sequential scan kernels. */
int64_t t2fw_lfw_default_ckpt_every(int64_t T, int64_t D, int64_t K, int dtype);
int64_t t2fw_lfw_ckpt_slots(int64_t T, int64_t ckpt_every);

/* Bytes of scratch (global memory beyond inputs and outputs, 256-byte aligned) that the
 * corresponding call needs for this problem; 0 means the scratch pointer may be NULL. */
size_t t2fw_lfw_forward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int dtype,
                                      int64_t ckpt_every);
size_t t2fw_lfw_backward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int dtype,
                                       int64_t ckpt_every);
size_t t2fw_dfw_forward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t M, int dtype);
size_t t2fw_dfw_backward_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t M, int dtype);

/*
 * Decay rule forward:  S_t = (f_t f_key_t^T) .* S_{t-1} + x_t k_t^T ,  o_t = S_t q_t.
 * Replaces torch.ops.lfw.forward = lfw_forward (t2fw/csrc/lfw.cpp:28-48), i.e. the scan
 * kernel lfw_cuda_forward (t2fw/csrc/lfw_kernel.cu:124-171) plus the einsum that forms the
 * outputs (t2fw/csrc/lfw.cpp:45).  Writes outputs and ckpt_states (both of `dtype`).
 */
int t2fw_lfw_forward(const void *x, const void *f, const void *q, const void *k,
                     const void *f_key, const void *state,
                     void *outputs, void *ckpt_states,
                     int64_t B, int64_t T, int64_t D, int64_t K, int dtype, int64_t ckpt_every,
                     void *scratch, size_t scratch_bytes, void *stream);

/*
 * Decay rule backward: all six gradients in forward-argument order.
 * Replaces torch.ops.lfw.backward = lfw_backward (t2fw/csrc/lfw.cpp:50-96), i.e. the reverse
 * scan lfw_cuda_backward (t2fw/csrc/lfw_kernel.cu:173-228), the five einsums and the two
 * in-place multiplies (t2fw/csrc/lfw.cpp:84-93).  `state` is the forward call's initial state
 * and `ckpt_states` the tensor the forward call wrote with the same ckpt_every.
 */
int t2fw_lfw_backward(const void *grad_output, const void *grad_state,
                      const void *x, const void *f, const void *q, const void *k,
                      const void *f_key, const void *state, const void *ckpt_states,
                      void *d_x, void *d_f, void *d_q, void *d_k, void *d_f_key, void *d_state,
                      int64_t B, int64_t T, int64_t D, int64_t K, int dtype, int64_t ckpt_every,
                      void *scratch, size_t scratch_bytes, void *stream);

/*
 * Fused decay-rule layer, d_head = 64 (additive; the reference has no counterpart: its wrapper
 * "assumes the input is already gated", t2fw/functional_lfw.py:26-29, and leaves the head fold, the
 * gate activation and the query scaling to the caller).
 *
 *   qkvg  [B, T, 4*H*64]  one row per (batch item, step): query | key | value | gate, each H*64
 *                         wide with head h at columns 64h .. 64h+63 - the output of the layer's
 *                         projection, read in place (no folded [B*H, T, 64] copies are made)
 *   state [B*H, 64, 64]   initial state per (batch item, head), row index b*H + h
 *   outputs [B, T, H*64]  heads already unfolded, ready for the output projection
 *   ckpt_states [B*H, ceil(T/64), 64, 64]; the last slot is the next state
 *
 * Computes, per (b, h), the decay rule with  x = value,  forget gate 1,  query scaled by 1/8
 * (= 1/sqrt(64)),  f_key = max(sigmoid(gate), 1/8).  The floor keeps every 32-step gate product
 * inside the range of the chunked kernels, so this entry point never needs the scan fallback.
 * The result equals t2fw_lfw_forward on the folded, activated tensors (rounded to the storage
 * type) bit for bit.  16-bit dtypes only; all pointers 16-byte aligned (T2FW_ERR_UNSUPPORTED
 * otherwise).  The backward returns d_qkvg [B, T, 4*H*64] (same layout, chain rule through the
 * activations included) and d_state.
 */
size_t t2fw_lfw_fused_scratch_bytes(int64_t B, int64_t T, int64_t H, int dtype);
int t2fw_lfw_fused_forward(const void *qkvg, const void *state, void *outputs, void *ckpt_states,
                           int64_t B, int64_t T, int64_t H, int dtype,
                           void *scratch, size_t scratch_bytes, void *stream);
int t2fw_lfw_fused_backward(const void *grad_output, const void *grad_state, const void *qkvg,
                            const void *state, const void *ckpt_states, void *d_qkvg, void *d_state,
                            int64_t B, int64_t T, int64_t H, int dtype,
                            void *scratch, size_t scratch_bytes, void *stream);

/* Summary of a sequence segment of the decay rule, for splitting the TIME axis over devices
 * (D = K = 64, 16-bit storage).  The recurrence is linear in the state, so a segment acts on the
 * state as  S_end = (decay_d decay_k^T) .* S_start + L  with the segment's total decays and the
 * state L that a zero state becomes; the state gradient runs backwards through the same map.
 *   backward = 0: (val_d, gate_d, val_k, gate_k) = (x, f, key, f_key) [B,T,64]; end_state = L
 *   backward = 1: (grad_output, f, query, f_key);  end_state = the state gradient at the segment
 *                 start for a zero gradient at its end
 * decay_d, decay_k: fp32 [B,64], products of f / f_key over the segment (NaN for a batch row whose
 * gate products leave the supported range).  Each device computes the summary of its own segment,
 * the devices exchange them ([B,64,64] + 2 x [B,64] each), combine the ones before (after) their own
 * into their incoming state (state gradient) and then call the ordinary forward (backward) entry
 * point: t2fw_b200/seq_parallel.py.  No counterpart in the reference, which has no multi-device
 * code; the recurrence it restates is t2fw/torch.py:21-28. */
size_t t2fw_lfw_segment_summary_scratch_bytes(int64_t B, int64_t T, int64_t D, int64_t K, int dtype);
int t2fw_lfw_segment_summary(int backward, const void *val_d, const void *gate_d, const void *val_k,
                             const void *gate_k, void *end_state, float *decay_d, float *decay_k, int64_t B,
                             int64_t T, int64_t D, int64_t K, int dtype, void *scratch, size_t scratch_bytes,
                             void *stream);

/* Fold of the exchanged segment summaries (one launch).  gathered: fp32 [n_segments][B][D*K + D + K],
 * per segment and batch row (end_state [D][K], decay_d [D], decay_k [K]) as t2fw_lfw_segment_summary
 * returns them (end_state converted to fp32); start, at_segment, total: fp32 [B][D][K].
 *   backward = 0: start = the state before step 0; at_segment = the state that enters `segment`
 *                 (segments 0 .. segment-1 applied in order); total (may be null) = the state after
 *                 the last segment
 *   backward = 1: start = the gradient of the final state; at_segment = the state gradient at the END
 *                 of `segment` (segments n_segments-1 .. segment+1 applied, last one first); total unused
 * No counterpart in the reference (no multi-device code); the recurrence is t2fw/torch.py:21-28. */
int t2fw_lfw_fold_summaries(int backward, const float *gathered, const float *start, float *at_segment,
                            float *total, int n_segments, int segment, int64_t B, int64_t D, int64_t K,
                            void *stream);

/*
 * Delta rule forward:  o_t = S_{t-1} q_t ,  delta_t = v_t - S_{t-1} k_t ,
 *                      S_t = S_{t-1} + delta_t k_t^T.
 * Replaces torch.ops.dfw.forward = lfw_forward (t2fw/csrc/dfw.cpp:27-39) and its kernel
 * (t2fw/csrc/dfw_kernel.cu:105-196, launcher :406-470).  `delta` ([B,T,D]) is kept for the
 * backward pass; it is float for 16- and 32-bit dtypes and double for T2FW_F64.
 */
int t2fw_dfw_forward(const void *q, const void *k, const void *v, const void *state,
                     void *outputs, void *final_state, void *delta,
                     int64_t B, int64_t T, int64_t D, int64_t M, int dtype, void *stream);

/*
 * Delta rule forward with caller-provided scratch (t2fw_dfw_forward_scratch_bytes): same
 * inputs, outputs and reference interface as t2fw_dfw_forward.  With scratch the library can run
 * the chunked tensor-core kernels (D = M = 64, 16-bit storage: per-chunk triangular solves in
 * fp32, chunk contractions on the tensor cores) instead of the step-by-step scan; the saved
 * `delta` is the same quantity either way, so either forward can be paired with the backward.
 */
int t2fw_dfw_forward_ws(const void *q, const void *k, const void *v, const void *state,
                        void *outputs, void *final_state, void *delta,
                        int64_t B, int64_t T, int64_t D, int64_t M, int dtype,
                        void *scratch, size_t scratch_bytes, void *stream);

/*
 * Delta rule backward: d_query, d_key, d_value, d_state.
 * Replaces torch.ops.dfw.backward = lfw_backward (t2fw/csrc/dfw.cpp:41-64) and its two
 * kernels (t2fw/csrc/dfw_kernel.cu:198-283 and :285-384, launcher :472-558).  Like the
 * reference it needs neither the values nor the initial state: it walks the state backwards
 * from final_state with the saved delta.
 */
int t2fw_dfw_backward(const void *grad_output, const void *grad_state,
                      const void *q, const void *k, const void *delta, const void *final_state,
                      void *d_q, void *d_k, void *d_v, void *d_state,
                      int64_t B, int64_t T, int64_t D, int64_t M, int dtype,
                      void *scratch, size_t scratch_bytes, void *stream);

/*
 * Delta rule backward without caller-provided scratch.  No counterpart in the reference
 * (its backward allocates freely through ATen).
 *
 * Same inputs and outputs as t2fw_dfw_backward and the same mathematical result; it always runs
 * the sequential scan kernels (never the chunked tensor-core kernels, which need far more
 * scratch), so on D = M = 64 16-bit problems it is an order of magnitude slower than
 * t2fw_dfw_backward and its rounding differs within the documented tolerance.  It is for hosts that cannot give the call
 * any device memory beyond the operator's own tensors and cannot call cudaMalloc themselves:
 * a runtime that reserved the entire GPU for its own pool when it started, a latency-critical
 * loop that must avoid the device-wide synchronisation an allocation implies, or a foreign
 * function bridge that only marshals an operator's inputs and outputs.  The float copy of
 * d_value that 16-bit problems need is kept in a 16 MiB array that is part of the library
 * image, so each GPU that uses the library carries it until the process ends.
 *
 * Limits and rules:
 *  - 16-bit dtypes: B*T*D <= t2fw_dfw_backward_noalloc_max_elems() (4 Mi elements), otherwise
 *    T2FW_ERR_SCRATCH with an explanatory message; 32- and 64-bit dtypes use no scratch and
 *    have no limit.
 *  - The first call on a device looks up the array's device address (with that device
 *    current); make that first call outside any stream capture.
 *  - The call allocates and frees nothing.  All calls on a device share the one array: it
 *    keeps whatever the previous call left (nothing in it has to start at zero, the row pass
 *    rewrites every element it later reads), and two calls that overlap on the GPU - from
 *    different streams or processes' threads - race on it.  Serialise them.
 */
size_t t2fw_dfw_backward_noalloc_max_elems(void);
int t2fw_dfw_backward_noalloc(const void *grad_output, const void *grad_state,
                              const void *q, const void *k, const void *delta,
                              const void *final_state,
                              void *d_q, void *d_k, void *d_v, void *d_state,
                              int64_t B, int64_t T, int64_t D, int64_t M, int dtype,
                              void *stream);

/*
 * Diagnostic: launches a one-warp kernel that waits, with a limit of `polls` polls, on a barrier
 * that nothing arrives on.  The wait runs out, the kernel sets *status (device int; NULL = the
 * library's own status word, the one t2fw_device_status reports) and returns: the give-up path of
 * the bounded waits with nothing in flight.  No counterpart in the reference.
 */
int t2fw_selftest_bounded_wait(int polls, int *status, void *stream);

/*
 * Diagnostic: D = A * B^T with the A operand [64 x 64] read from tensor memory (written there by
 * tcgen05.st, stored in both lane sets) and B [64 x 64] a 128-byte-swizzle shared-memory tile: the
 * operand forms of the decay rule's 64-step chunk kernels.  All row-major fp32 device arrays, used
 * at TF32 precision.  *status (device int) is set to 1 if a bounded wait expired.  No counterpart
 * in the reference.
 */
int t2fw_selftest_umma_ts(const float *A, const float *B, float *D, int *status, void *stream);

/*
 * Diagnostic: exercises the tensor-core building blocks of the chunked kernels in isolation
 * (tensor-memory allocation, shared-memory matrix descriptors in both operand orientations,
 * tcgen05.mma, completion tracking, accumulator loads).  No counterpart in the reference.
 * Computes D1 = A1 * B1^T and D2 = A2 * B2^T with A [64 x Kc], B [N x Kc], D [64 x N], all
 * row-major fp32 device arrays (operands are used at TF32 precision).  a_mn / b_mn must be 0:
 * TF32 operands are K-major only in the un-swizzled shared-memory form.  *status (device int)
 * is set to 1 if a bounded wait expired.  N, Kc: multiples of 8 in [8, 64].
 */
int t2fw_selftest_umma(const float *A1, const float *B1, const float *A2, const float *B2,
                       float *D1, float *D2, int N, int Kc, int a_mn, int b_mn, int *status,
                       void *stream);

/* Same diagnostic with bf16 operands (rounded from the fp32 inputs inside the kernel); here both
 * operand orientations exist, a_mn / b_mn in {0, 1}.  Kc: multiple of 16 in [16, 64]. */
int t2fw_selftest_umma16(const float *A1, const float *B1, const float *A2, const float *B2,
                         float *D1, float *D2, int N, int Kc, int a_mn, int b_mn, int *status,
                         void *stream);

#ifdef __cplusplus
}
#endif
#endif /* T2FW_B200_H */
