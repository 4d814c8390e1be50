"""The decay rule with the TIME axis of one long sequence split over the ranks of a process group.

The path shards by batch x head without any exchange (t2fw_b200/parallel.py); this module is for
the case of fewer rows than devices and very long sequences.  Rank r holds steps
[r * T/G, (r + 1) * T/G) of every batch row.  The recurrence (t2fw/torch.py:21-28 of the reference)
is linear in the state, so a segment acts on the state as

    S_end = (A G^T) .* S_start + L        A, G = products of f / f_key over the segment,
                                          L    = the state a zero state becomes over the segment

and the state gradient runs backwards through the same map.  One call therefore is

    forward:   summary of the own segment (two cheap kernels)  ->  ONE all-gather of the summaries
               ([B,64,64] + 2 x [B,64] floats per rank, received into local memory)  ->  fold of
               the ranks before this one into the incoming state (one kernel: torch.ops.lfw.fold_summaries;
               the CPU ranks of the tests fold with tensor operations)  ->  the ordinary forward kernels
    backward:  the same with the summaries of the output gradients, folded from the last rank down.

No kernel reads another device's memory; the only collectives are the two all-gathers (and one
all-reduce of the final state's gradient).  The per-segment work goes through an `ops` object so that
the exchange and fold logic can be tested on CPU ranks (gloo) with the step-by-step oracle doing the
segment work; `CudaSegmentOps` is the product path (D = K = 64, fp16 / bf16).
"""
import torch
import torch.distributed as dist


class CudaSegmentOps:
    """Segment work on the CUDA kernels (torch.ops.lfw.*)."""

    def __init__(self):
        from . import _lib

        _lib.load_ops()

    def summary(self, val_d, gate_d, val_k, gate_k, backward):
        return torch.ops.lfw.segment_summary(val_d, gate_d, val_k, gate_k, backward)

    def fold(self, gathered, start32, segment, backward):
        """gathered [world, B, D*K+D+K] fp32 -> [state entering `segment`, state after the last segment]
        (backward: [state gradient at the end of `segment`]), one launch."""
        return torch.ops.lfw.fold_summaries(gathered, start32, segment, backward)

    def forward(self, x, f, q, k, fk, state):
        return torch.ops.lfw.forward(x, f, q, k, fk, state)

    def backward(self, go, gs, x, f, q, k, fk, out, state, ckpt):
        return torch.ops.lfw.backward(go, gs, x, f, q, k, fk, out, state, ckpt)


def _acc(dtype):
    """Summaries are exchanged and folded in fp32 (fp64 for fp64 tensors)."""
    return torch.float64 if dtype == torch.float64 else torch.float32


def pack_summary(end_state, decay_d, decay_k):
    """[B, D*K + D + K]: what one rank contributes to the exchange."""
    B, acc = end_state.shape[0], _acc(end_state.dtype)
    return torch.cat([end_state.to(acc).reshape(B, -1), decay_d.to(acc), decay_k.to(acc)], dim=1).contiguous()


def unpack_summary(buf, D, K):
    B = buf.shape[0]
    return buf[:, :D * K].reshape(B, D, K), buf[:, D * K:D * K + D], buf[:, D * K + D:]


def fold_forward(state, summaries, upto, D, K):
    """State at the start of segment `upto`: segments 0 .. upto-1 applied to `state`."""
    S = state.to(_acc(state.dtype))
    for j in range(upto):
        L, A, G = unpack_summary(summaries[j], D, K)
        S = (A[:, :, None] * G[:, None, :]) * S + L
    return S


def fold_backward(grad_final, summaries, after, D, K):
    """State gradient at the END of segment `after`: the segments behind it applied, last one first,
    to the gradient of the final state.  summaries[j] = (local gradient at the start of j, A_j, G_j)."""
    R = grad_final.to(_acc(grad_final.dtype))
    for j in range(len(summaries) - 1, after, -1):
        Gb, A, G = unpack_summary(summaries[j], D, K)
        R = (A[:, :, None] * G[:, None, :]) * R + Gb
    return R


def all_gather_summaries(buf, group):
    """[world, B, N]: every rank's packed summary, received into one local tensor."""
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(buf.shape), dtype=buf.dtype, device=buf.device)
    dist.all_gather(list(out.unbind(0)), buf, group=group)
    return out


class LFWSeqParallelFunction(torch.autograd.Function):
    """`apply(value, forget, query, key, f_key, state, group=None, ops=None) -> (outputs, final_state)`

    value .. f_key are this rank's segment [B, T_r, .] (segments in rank order make up the
    sequence; they may differ in length), `state` [B, D, K] is the state before step 0 of the WHOLE
    sequence, the same on every rank.  outputs is this rank's segment of the outputs; final_state is
    the state after the whole sequence, the same on every rank.  Gradients: each rank gets the
    gradients of its own segment; d_state is returned on rank 0 (zeros elsewhere, so that a sum over
    ranks is the gradient of the replicated input); the gradient of final_state is summed over ranks."""

    @staticmethod
    def forward(ctx, value, forget, query, key, f_key, state, group=None, ops=None):
        ops = ops if ops is not None else CudaSegmentOps()
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        D, K = value.shape[2], key.shape[2]
        x, f, q, k, fk = (t.contiguous() for t in (value, forget, query, key, f_key))
        if world == 1:      # nothing to exchange: the ordinary call, its last checkpoint is the final state
            s_in = state.contiguous()
            outputs, ckpt = ops.forward(x, f, q, k, fk, s_in)
            ctx.save_for_backward(x, f, q, k, fk, outputs, s_in, ckpt)
            ctx.group, ctx.ops, ctx.dims = group, ops, (D, K)
            return outputs, ckpt[:, -1].clone()
        L, A, G = ops.summary(x, f, k, fk, False)
        summaries = all_gather_summaries(pack_summary(L, A, G), group)
        if hasattr(ops, "fold"):
            s_in32, final32 = ops.fold(summaries, state.to(_acc(state.dtype)).contiguous(), rank, False)
        else:
            s_in32 = fold_forward(state, summaries, rank, D, K)
            # the state after the whole sequence: carry on from this rank's incoming state
            final32 = fold_forward(s_in32, summaries[rank:], world - rank, D, K)
        s_in = s_in32.to(state.dtype).contiguous()
        outputs, ckpt = ops.forward(x, f, q, k, fk, s_in)
        final = final32.to(state.dtype)
        ctx.save_for_backward(x, f, q, k, fk, outputs, s_in, ckpt, summaries[rank])
        ctx.group, ctx.ops, ctx.dims = group, ops, (D, K)
        return outputs, final

    @staticmethod
    def backward(ctx, grad_output, grad_final):
        group, ops, (D, K) = ctx.group, ctx.ops, ctx.dims
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        go = grad_output.contiguous()
        if world == 1:
            x, f, q, k, fk, outputs, s_in, ckpt = ctx.saved_tensors
            grads = ops.backward(go, grad_final.to(s_in.dtype).contiguous(), x, f, q, k, fk, outputs, s_in, ckpt)
            return (*grads, None, None)
        x, f, q, k, fk, outputs, s_in, ckpt, own_summary = ctx.saved_tensors
        g_final = grad_final.to(_acc(grad_final.dtype)).contiguous()
        dist.all_reduce(g_final, group=group)      # every rank may have used final_state
        Gb, _, _ = ops.summary(go, f, q, fk, True)
        # the decays of a segment are the same in both directions: take them from the forward exchange
        _, A, G = unpack_summary(own_summary, D, K)
        summaries = all_gather_summaries(pack_summary(Gb, A, G), group)
        if hasattr(ops, "fold"):
            r_end32 = ops.fold(summaries, g_final, rank, True)[0]
        else:
            r_end32 = fold_backward(g_final, summaries, rank, D, K)
        r_end = r_end32.to(s_in.dtype).contiguous()
        d_x, d_f, d_q, d_k, d_fk, d_s = ops.backward(go, r_end, x, f, q, k, fk, outputs, s_in, ckpt)
        if rank != 0:
            d_s = torch.zeros_like(d_s)
        return d_x, d_f, d_q, d_k, d_fk, d_s, None, None
