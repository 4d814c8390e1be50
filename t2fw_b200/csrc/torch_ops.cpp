// PyTorch operator library: torch.ops.lfw.{forward,backward} and torch.ops.dfw.{forward,backward}
// with the schemas of the reference's op libraries (t2fw/csrc/lfw.cpp:98-101,
// t2fw/csrc/dfw.cpp:66-69).  This file is only an adapter: it validates tensors, allocates the
// outputs (and scratch) with the caching allocator, picks the caller's device and current
// stream, and forwards raw pointers to the C ABI in include/t2fw_b200.h.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstdlib>
#include <vector>

#include "t2fw_b200.h"

namespace {

#define T2FW_CHECK_INPUT(x)                                             \
  TORCH_CHECK((x).device().is_cuda(), #x " must be a CUDA tensor");     \
  TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")

int dtype_code(const at::Tensor &t) {
  switch (t.scalar_type()) {
    case at::kHalf: return T2FW_F16;
    case at::kBFloat16: return T2FW_BF16;
    case at::kFloat: return T2FW_F32;
    case at::kDouble: return T2FW_F64;
    default: TORCH_CHECK(false, "t2fw: unsupported dtype ", t.scalar_type());
  }
  return -1;
}

void check_status(int rc, const char *what) {
  TORCH_CHECK(rc == T2FW_OK, what, " failed (status ", rc, "): ", t2fw_last_error());
}

void check_same(const at::Tensor &a, const at::Tensor &ref, const char *name) {
  TORCH_CHECK(a.scalar_type() == ref.scalar_type(), name, ": dtype differs from the first tensor's");
  TORCH_CHECK(a.device() == ref.device(), name, ": device differs from the first tensor's");
}

int64_t ckpt_interval(int64_t T, int64_t D, int64_t K, int dtype) {
  if (const char *e = std::getenv("T2FW_CKPT_EVERY")) {
    const long v = std::atol(e);
    if (v > 0) return v;
  }
  return t2fw_lfw_default_ckpt_every(T, D, K, dtype);
}

at::Tensor make_scratch(size_t bytes, const at::Tensor &like) {
  if (bytes == 0) return at::Tensor();
  return at::empty({(int64_t)bytes}, like.options().dtype(at::kByte));
}

void *ptr_or_null(const at::Tensor &t) { return t.defined() ? t.data_ptr() : nullptr; }

// ---- decay rule ---------------------------------------------------------------------------
std::vector<at::Tensor> lfw_forward(at::Tensor x, at::Tensor f, at::Tensor query, at::Tensor key,
                                    at::Tensor f_key, at::Tensor state) {
  T2FW_CHECK_INPUT(x);
  T2FW_CHECK_INPUT(f);
  T2FW_CHECK_INPUT(query);
  T2FW_CHECK_INPUT(key);
  T2FW_CHECK_INPUT(f_key);
  T2FW_CHECK_INPUT(state);
  TORCH_CHECK(x.dim() == 3 && query.dim() == 3 && state.dim() == 3, "expected x [B,T,D], query [B,T,K], state [B,D,K]");
  const int64_t B = x.size(0), T = x.size(1), D = x.size(2), K = query.size(2);
  TORCH_CHECK(f.sizes() == x.sizes(), "f must have x's shape");
  TORCH_CHECK(query.size(0) == B && query.size(1) == T, "query must be [B,T,K]");
  TORCH_CHECK(key.sizes() == query.sizes() && f_key.sizes() == query.sizes(), "key and f_key must have query's shape");
  TORCH_CHECK(state.size(0) == B && state.size(1) == D && state.size(2) == K, "state must be [B,D,K]");
  check_same(f, x, "f"); check_same(query, x, "query"); check_same(key, x, "key");
  check_same(f_key, x, "f_key"); check_same(state, x, "state");
  TORCH_CHECK(B > 0 && T > 0 && D > 0 && K > 0, "empty tensors are not supported");

  const c10::cuda::CUDAGuard guard(x.device());
  const int dt = dtype_code(x);
  const int64_t C = ckpt_interval(T, D, K, dt);
  const int64_t slots = t2fw_lfw_ckpt_slots(T, C);
  at::Tensor outputs = at::empty({B, T, D}, x.options());
  at::Tensor ckpt = at::empty({B, slots, D, K}, x.options());
  const size_t sb = t2fw_lfw_forward_scratch_bytes(B, T, D, K, dt, C);
  at::Tensor scratch = make_scratch(sb, x);
  auto stream = at::cuda::getCurrentCUDAStream();
  check_status(t2fw_lfw_forward(x.data_ptr(), f.data_ptr(), query.data_ptr(), key.data_ptr(),
                                f_key.data_ptr(), state.data_ptr(), outputs.data_ptr(),
                                ckpt.data_ptr(), B, T, D, K, dt, C, ptr_or_null(scratch), sb,
                                stream.stream()),
               "lfw.forward");
  return {outputs, ckpt};
}

std::vector<at::Tensor> lfw_backward(at::Tensor grad_output, at::Tensor grad_state,
                                     at::Tensor value, at::Tensor forget, at::Tensor query,
                                     at::Tensor key, at::Tensor f_key, at::Tensor outputs,
                                     at::Tensor state, at::Tensor ckpt_states) {
  T2FW_CHECK_INPUT(grad_output);
  T2FW_CHECK_INPUT(grad_state);
  T2FW_CHECK_INPUT(value);
  T2FW_CHECK_INPUT(forget);
  T2FW_CHECK_INPUT(query);
  T2FW_CHECK_INPUT(key);
  T2FW_CHECK_INPUT(f_key);
  T2FW_CHECK_INPUT(outputs);
  T2FW_CHECK_INPUT(state);
  T2FW_CHECK_INPUT(ckpt_states);
  TORCH_CHECK(value.dim() == 3 && query.dim() == 3 && state.dim() == 3 && ckpt_states.dim() == 4, "bad ranks");
  const int64_t B = value.size(0), T = value.size(1), D = value.size(2), K = query.size(2);
  TORCH_CHECK(grad_output.sizes() == value.sizes(), "grad_output must be [B,T,D]");
  TORCH_CHECK(forget.sizes() == value.sizes() && outputs.sizes() == value.sizes(), "forget and outputs must be [B,T,D]");
  TORCH_CHECK(query.size(0) == B && query.size(1) == T, "query must be [B,T,K]");
  TORCH_CHECK(key.sizes() == query.sizes() && f_key.sizes() == query.sizes(), "key and f_key must have query's shape");
  TORCH_CHECK(state.size(0) == B && state.size(1) == D && state.size(2) == K, "state must be [B,D,K]");
  TORCH_CHECK(grad_state.sizes() == state.sizes(), "grad_state must be [B,D,K]");
  check_same(grad_output, value, "grad_output"); check_same(grad_state, value, "grad_state");
  check_same(forget, value, "forget"); check_same(query, value, "query"); check_same(key, value, "key");
  check_same(f_key, value, "f_key"); check_same(outputs, value, "outputs"); check_same(state, value, "state");
  check_same(ckpt_states, value, "ckpt_states");
  TORCH_CHECK(B > 0 && T > 0 && D > 0 && K > 0, "empty tensors are not supported");

  const c10::cuda::CUDAGuard guard(value.device());
  const int dt = dtype_code(value);
  const int64_t C = ckpt_interval(T, D, K, dt);
  TORCH_CHECK(ckpt_states.size(0) == B && ckpt_states.size(1) == t2fw_lfw_ckpt_slots(T, C) &&
                  ckpt_states.size(2) == D && ckpt_states.size(3) == K,
              "ckpt_states does not match the checkpoint interval in use");
  // separate allocations: views of one buffer would be flagged by autograd when a caller later
  // modifies a gradient in place
  at::Tensor d_x = at::empty_like(value), d_f = at::empty_like(forget);
  at::Tensor d_q = at::empty_like(query), d_k = at::empty_like(key), d_fk = at::empty_like(f_key);
  at::Tensor d_s = at::empty_like(state);
  const size_t sb = t2fw_lfw_backward_scratch_bytes(B, T, D, K, dt, C);
  at::Tensor scratch = make_scratch(sb, value);
  auto stream = at::cuda::getCurrentCUDAStream();
  check_status(t2fw_lfw_backward(grad_output.data_ptr(), grad_state.data_ptr(), value.data_ptr(),
                                 forget.data_ptr(), query.data_ptr(), key.data_ptr(),
                                 f_key.data_ptr(), state.data_ptr(), ckpt_states.data_ptr(),
                                 d_x.data_ptr(), d_f.data_ptr(), d_q.data_ptr(), d_k.data_ptr(),
                                 d_fk.data_ptr(), d_s.data_ptr(), B, T, D, K, dt, C,
                                 ptr_or_null(scratch), sb, stream.stream()),
               "lfw.backward");
  return {d_x, d_f, d_q, d_k, d_fk, d_s};
}

// One decode step (T = 1) into caller-owned buffers: outputs [B,1,D] and state_out [B,D,K] are
// written, nothing is allocated, so a loop that alternates two state buffers can be captured in a
// CUDA graph and replayed.  Additive: the reference has no counterpart (its recurrent use is
// LFWFunction.apply with the returned state fed back, t2fw/functional_lfw.py:65).
void lfw_decode_step(at::Tensor x, at::Tensor f, at::Tensor query, at::Tensor key, at::Tensor f_key,
                     at::Tensor state_in, at::Tensor state_out, at::Tensor outputs) {
  T2FW_CHECK_INPUT(x);
  T2FW_CHECK_INPUT(f);
  T2FW_CHECK_INPUT(query);
  T2FW_CHECK_INPUT(key);
  T2FW_CHECK_INPUT(f_key);
  T2FW_CHECK_INPUT(state_in);
  T2FW_CHECK_INPUT(state_out);
  T2FW_CHECK_INPUT(outputs);
  TORCH_CHECK(x.dim() == 3 && x.size(1) == 1 && query.dim() == 3 && state_in.dim() == 3,
              "expected x [B,1,D], query [B,1,K], state [B,D,K]");
  const int64_t B = x.size(0), D = x.size(2), K = query.size(2);
  TORCH_CHECK(f.sizes() == x.sizes() && outputs.sizes() == x.sizes(), "f and outputs must have x's shape");
  TORCH_CHECK(query.size(0) == B && query.size(1) == 1, "query must be [B,1,K]");
  TORCH_CHECK(key.sizes() == query.sizes() && f_key.sizes() == query.sizes(), "key and f_key must have query's shape");
  TORCH_CHECK(state_in.size(0) == B && state_in.size(1) == D && state_in.size(2) == K, "state_in must be [B,D,K]");
  TORCH_CHECK(state_out.sizes() == state_in.sizes(), "state_out must have state_in's shape");
  TORCH_CHECK(state_out.data_ptr() != state_in.data_ptr(), "state_out must not be state_in: alternate two buffers");
  check_same(f, x, "f"); check_same(query, x, "query"); check_same(key, x, "key"); check_same(f_key, x, "f_key");
  check_same(state_in, x, "state_in"); check_same(state_out, x, "state_out"); check_same(outputs, x, "outputs");
  TORCH_CHECK(B > 0 && D > 0 && K > 0, "empty tensors are not supported");
  const c10::cuda::CUDAGuard guard(x.device());
  const int dt = dtype_code(x);
  auto stream = at::cuda::getCurrentCUDAStream();
  // T = 1: one checkpoint slot, which is the new state
  check_status(t2fw_lfw_forward(x.data_ptr(), f.data_ptr(), query.data_ptr(), key.data_ptr(), f_key.data_ptr(),
                                state_in.data_ptr(), outputs.data_ptr(), state_out.data_ptr(), B, 1, D, K, dt, 1,
                                nullptr, 0, stream.stream()),
               "lfw.decode_step");
}

// Fused decay-rule layer (d_head = 64): heads are read in place from the projection output
// qkvg [B,T,4*H*64] = query | key | value | gate; returns {outputs [B,T,H*64], ckpt_states}.
std::vector<at::Tensor> lfw_fused_forward(at::Tensor qkvg, at::Tensor state, int64_t n_head) {
  T2FW_CHECK_INPUT(qkvg);
  T2FW_CHECK_INPUT(state);
  TORCH_CHECK(qkvg.dim() == 3 && state.dim() == 3 && n_head > 0, "expected qkvg [B,T,4*H*64], state [B*H,64,64]");
  const int64_t B = qkvg.size(0), T = qkvg.size(1), H = n_head;
  TORCH_CHECK(qkvg.size(2) == 4 * H * 64, "qkvg must be [B,T,4*H*64]");
  TORCH_CHECK(state.size(0) == B * H && state.size(1) == 64 && state.size(2) == 64, "state must be [B*H,64,64]");
  check_same(state, qkvg, "state");
  TORCH_CHECK(B > 0 && T > 0, "empty tensors are not supported");
  const c10::cuda::CUDAGuard guard(qkvg.device());
  const int dt = dtype_code(qkvg);
  at::Tensor outputs = at::empty({B, T, H * 64}, qkvg.options());
  at::Tensor ckpt = at::empty({B * H, t2fw_lfw_ckpt_slots(T, 64), 64, 64}, qkvg.options());
  const size_t sb = t2fw_lfw_fused_scratch_bytes(B, T, H, dt);
  at::Tensor scratch = make_scratch(sb, qkvg);
  auto stream = at::cuda::getCurrentCUDAStream();
  check_status(t2fw_lfw_fused_forward(qkvg.data_ptr(), state.data_ptr(), outputs.data_ptr(), ckpt.data_ptr(), B, T, H,
                                      dt, ptr_or_null(scratch), sb, stream.stream()),
               "lfw.fused_forward");
  return {outputs, ckpt};
}

std::vector<at::Tensor> lfw_fused_backward(at::Tensor grad_output, at::Tensor grad_state, at::Tensor qkvg,
                                           at::Tensor state, at::Tensor ckpt_states, int64_t n_head) {
  T2FW_CHECK_INPUT(grad_output);
  T2FW_CHECK_INPUT(grad_state);
  T2FW_CHECK_INPUT(qkvg);
  T2FW_CHECK_INPUT(state);
  T2FW_CHECK_INPUT(ckpt_states);
  TORCH_CHECK(qkvg.dim() == 3 && state.dim() == 3 && grad_output.dim() == 3 && ckpt_states.dim() == 4 && n_head > 0,
              "bad ranks");
  const int64_t B = qkvg.size(0), T = qkvg.size(1), H = n_head;
  TORCH_CHECK(qkvg.size(2) == 4 * H * 64, "qkvg must be [B,T,4*H*64]");
  TORCH_CHECK(grad_output.size(0) == B && grad_output.size(1) == T && grad_output.size(2) == H * 64,
              "grad_output must be [B,T,H*64]");
  TORCH_CHECK(state.size(0) == B * H && state.size(1) == 64 && state.size(2) == 64, "state must be [B*H,64,64]");
  TORCH_CHECK(grad_state.sizes() == state.sizes(), "grad_state must have state's shape");
  TORCH_CHECK(ckpt_states.size(0) == B * H && ckpt_states.size(1) == t2fw_lfw_ckpt_slots(T, 64) &&
                  ckpt_states.size(2) == 64 && ckpt_states.size(3) == 64,
              "ckpt_states must be the tensor lfw.fused_forward returned");
  check_same(grad_output, qkvg, "grad_output"); check_same(grad_state, qkvg, "grad_state");
  check_same(state, qkvg, "state"); check_same(ckpt_states, qkvg, "ckpt_states");
  const c10::cuda::CUDAGuard guard(qkvg.device());
  const int dt = dtype_code(qkvg);
  at::Tensor d_qkvg = at::empty_like(qkvg), d_state = at::empty_like(state);
  const size_t sb = t2fw_lfw_fused_scratch_bytes(B, T, H, dt);
  at::Tensor scratch = make_scratch(sb, qkvg);
  auto stream = at::cuda::getCurrentCUDAStream();
  check_status(t2fw_lfw_fused_backward(grad_output.data_ptr(), grad_state.data_ptr(), qkvg.data_ptr(), state.data_ptr(),
                                       ckpt_states.data_ptr(), d_qkvg.data_ptr(), d_state.data_ptr(), B, T, H, dt,
                                       ptr_or_null(scratch), sb, stream.stream()),
               "lfw.fused_backward");
  return {d_qkvg, d_state};
}

// ---- delta rule ---------------------------------------------------------------------------
at::ScalarType acc_type(const at::Tensor &t) {
  return t.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
}

std::vector<at::Tensor> dfw_forward(at::Tensor query, at::Tensor key, at::Tensor value,
                                    at::Tensor state) {
  T2FW_CHECK_INPUT(query);
  T2FW_CHECK_INPUT(key);
  T2FW_CHECK_INPUT(value);
  T2FW_CHECK_INPUT(state);
  TORCH_CHECK(value.dim() == 3 && query.dim() == 3 && state.dim() == 3, "expected value [B,T,D], query [B,T,M], state [B,D,M]");
  const int64_t B = value.size(0), T = value.size(1), D = value.size(2), M = query.size(2);
  TORCH_CHECK(query.size(0) == B && query.size(1) == T && key.sizes() == query.sizes(), "query/key must be [B,T,M]");
  TORCH_CHECK(state.size(0) == B && state.size(1) == D && state.size(2) == M, "state must be [B,D,M]");
  check_same(query, value, "query"); check_same(key, value, "key"); check_same(state, value, "state");
  TORCH_CHECK(B > 0 && T > 0 && D > 0 && M > 0, "empty tensors are not supported");

  const c10::cuda::CUDAGuard guard(value.device());
  const int dt = dtype_code(value);
  at::Tensor outputs = at::empty_like(value);
  at::Tensor final_state = at::empty_like(state);
  at::Tensor delta = at::empty({B, T, D}, value.options().dtype(acc_type(value)));
  auto stream = at::cuda::getCurrentCUDAStream();
  const size_t sb = t2fw_dfw_forward_scratch_bytes(B, T, D, M, dt);
  at::Tensor scratch;
  if (sb) scratch = at::empty({(int64_t)sb}, value.options().dtype(at::kByte));
  check_status(t2fw_dfw_forward_ws(query.data_ptr(), key.data_ptr(), value.data_ptr(),
                                   state.data_ptr(), outputs.data_ptr(), final_state.data_ptr(),
                                   delta.data_ptr(), B, T, D, M, dt, sb ? scratch.data_ptr() : nullptr, sb,
                                   stream.stream()),
               "dfw.forward");
  return {outputs, final_state, delta};
}

std::vector<at::Tensor> dfw_backward(at::Tensor grad_output, at::Tensor grad_state,
                                     at::Tensor query, at::Tensor key, at::Tensor delta_value,
                                     at::Tensor final_state) {
  T2FW_CHECK_INPUT(grad_output);
  T2FW_CHECK_INPUT(grad_state);
  T2FW_CHECK_INPUT(query);
  T2FW_CHECK_INPUT(key);
  T2FW_CHECK_INPUT(delta_value);
  T2FW_CHECK_INPUT(final_state);
  TORCH_CHECK(grad_output.dim() == 3 && query.dim() == 3 && final_state.dim() == 3, "bad ranks");
  const int64_t B = grad_output.size(0), T = grad_output.size(1), D = grad_output.size(2),
                M = query.size(2);
  TORCH_CHECK(delta_value.sizes() == grad_output.sizes(), "delta_value must be [B,T,D]");
  TORCH_CHECK(query.size(0) == B && query.size(1) == T && key.sizes() == query.sizes(), "query/key must be [B,T,M]");
  TORCH_CHECK(final_state.size(0) == B && final_state.size(1) == D && final_state.size(2) == M, "final_state must be [B,D,M]");
  TORCH_CHECK(grad_state.sizes() == final_state.sizes(), "grad_state must be [B,D,M]");
  check_same(key, query, "key");
  TORCH_CHECK(delta_value.device() == query.device(), "delta_value: device differs from query's");
  TORCH_CHECK(B > 0 && T > 0 && D > 0 && M > 0, "empty tensors are not supported");
  TORCH_CHECK(delta_value.scalar_type() == acc_type(query), "delta_value must be the tensor dfw.forward returned");
  check_same(grad_output, query, "grad_output"); check_same(grad_state, query, "grad_state");
  check_same(final_state, query, "final_state");

  const c10::cuda::CUDAGuard guard(query.device());
  const int dt = dtype_code(query);
  at::Tensor d_q = at::empty_like(query), d_k = at::empty_like(key);
  at::Tensor d_v = at::empty_like(grad_output), d_s = at::empty_like(final_state);
  const size_t sb = t2fw_dfw_backward_scratch_bytes(B, T, D, M, dt);
  at::Tensor scratch = make_scratch(sb, query);
  auto stream = at::cuda::getCurrentCUDAStream();
  check_status(t2fw_dfw_backward(grad_output.data_ptr(), grad_state.data_ptr(), query.data_ptr(),
                                 key.data_ptr(), delta_value.data_ptr(), final_state.data_ptr(),
                                 d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_s.data_ptr(), B,
                                 T, D, M, dt, ptr_or_null(scratch), sb, stream.stream()),
               "dfw.backward");
  return {d_q, d_k, d_v, d_s};
}

// What a sequence segment does to the state (backward = false: inputs value, forget, key, f_key) or
// to the state gradient (backward = true: grad_output, forget, query, f_key), D = K = 64, 16-bit:
// {end_state [B,64,64], decay_d [B,64] fp32, decay_k [B,64] fp32}.  See t2fw_lfw_segment_summary.
std::vector<at::Tensor> lfw_segment_summary(at::Tensor val_d, at::Tensor gate_d, at::Tensor val_k, at::Tensor gate_k,
                                            bool backward) {
  T2FW_CHECK_INPUT(val_d);
  T2FW_CHECK_INPUT(gate_d);
  T2FW_CHECK_INPUT(val_k);
  T2FW_CHECK_INPUT(gate_k);
  TORCH_CHECK(val_d.dim() == 3 && val_k.dim() == 3, "expected [B,T,D] and [B,T,K] tensors");
  const int64_t B = val_d.size(0), T = val_d.size(1), D = val_d.size(2), K = val_k.size(2);
  TORCH_CHECK(gate_d.sizes() == val_d.sizes() && gate_k.sizes() == val_k.sizes() && val_k.size(0) == B &&
                  val_k.size(1) == T,
              "segment_summary: tensor shapes do not agree");
  check_same(gate_d, val_d, "gate_d");
  check_same(val_k, val_d, "val_k");
  check_same(gate_k, val_d, "gate_k");
  TORCH_CHECK(B > 0 && T > 0, "empty tensors are not supported");
  const c10::cuda::CUDAGuard guard(val_d.device());
  const int dt = dtype_code(val_d);
  at::Tensor end_state = at::empty({B, D, K}, val_d.options());
  at::Tensor decay_d = at::empty({B, D}, val_d.options().dtype(at::kFloat));
  at::Tensor decay_k = at::empty({B, K}, val_d.options().dtype(at::kFloat));
  const size_t sb = t2fw_lfw_segment_summary_scratch_bytes(B, T, D, K, dt);
  TORCH_CHECK(sb != 0, "lfw.segment_summary: D = K = 64 and fp16 / bf16 only");
  at::Tensor scratch = make_scratch(sb, val_d);
  auto stream = at::cuda::getCurrentCUDAStream();
  check_status(t2fw_lfw_segment_summary(backward ? 1 : 0, val_d.data_ptr(), gate_d.data_ptr(), val_k.data_ptr(),
                                        gate_k.data_ptr(), end_state.data_ptr(), decay_d.data_ptr<float>(),
                                        decay_k.data_ptr<float>(), B, T, D, K, dt, ptr_or_null(scratch), sb,
                                        stream.stream()),
               "lfw.segment_summary");
  return {end_state, decay_d, decay_k};
}

// Fold of gathered segment summaries [n][B][D*K+D+K] (fp32) over `start` [B,D,K] (fp32):
// {state entering segment `segment`, state after the last segment} (backward = false) or
// {state gradient at the end of `segment`} (backward = true).  See t2fw_lfw_fold_summaries.
std::vector<at::Tensor> lfw_fold_summaries(at::Tensor gathered, at::Tensor start, int64_t segment, bool backward) {
  T2FW_CHECK_INPUT(gathered);
  T2FW_CHECK_INPUT(start);
  TORCH_CHECK(gathered.scalar_type() == at::kFloat && start.scalar_type() == at::kFloat,
              "fold_summaries: fp32 tensors expected");
  TORCH_CHECK(gathered.dim() == 3 && start.dim() == 3, "fold_summaries: expected [n,B,D*K+D+K] and [B,D,K]");
  const int64_t n = gathered.size(0), B = start.size(0), D = start.size(1), K = start.size(2);
  TORCH_CHECK(gathered.size(1) == B && gathered.size(2) == D * K + D + K && gathered.device() == start.device(),
              "fold_summaries: tensor shapes or devices do not agree");
  TORCH_CHECK(n > 0 && n < (1 << 20) && segment >= 0 && segment < n, "fold_summaries: segment out of range");
  const c10::cuda::CUDAGuard guard(start.device());
  at::Tensor at_seg = at::empty_like(start);
  at::Tensor total = backward ? at::Tensor() : at::empty_like(start);
  auto stream = at::cuda::getCurrentCUDAStream();
  check_status(t2fw_lfw_fold_summaries(backward ? 1 : 0, gathered.data_ptr<float>(), start.data_ptr<float>(),
                                       at_seg.data_ptr<float>(), backward ? nullptr : total.data_ptr<float>(), (int)n,
                                       (int)segment, B, D, K, stream.stream()),
               "lfw.fold_summaries");
  if (backward) return {at_seg};
  return {at_seg, total};
}

}  // namespace

TORCH_LIBRARY(lfw, m) {
  m.def("forward", lfw_forward);
  m.def("backward", lfw_backward);
  m.def("decode_step", lfw_decode_step);
  m.def("fused_forward", lfw_fused_forward);
  m.def("fused_backward", lfw_fused_backward);
  m.def("segment_summary", lfw_segment_summary);
  m.def("fold_summaries", lfw_fold_summaries);
}

TORCH_LIBRARY(dfw, m) {
  m.def("forward", dfw_forward);
  m.def("backward", dfw_backward);
}
