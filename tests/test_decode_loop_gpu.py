"""Recurrent use of the decay rule: the state of a chunked (T > 1) call handed to T = 1 steps, the
allocation-free decode step and the graph-replayed decode loop, and the autograd wrapper under
CUDA-graph capture.  Reference protocol: the returned state is fed to the next call
(t2fw/functional_lfw.py:65); its benchmark times that step (tests/benchmark.py:104-105)."""
import pytest
import torch

from helpers import GRAD_TOL, OUT_TOL, lfw_inputs, max_rel_err, to_dev
from oracle import fw_oracle

pytestmark = pytest.mark.gpu


def test_chunked_prefill_state_feeds_decode_steps(cuda):
    """State from a T = 1024 call on the tensor-core path, then six T = 1 steps through the decode
    loop (the first trip eager, the rest replayed from the graph), against the oracle on T = 1030."""
    from t2fw_b200.decode import LFWDecodeLoop
    from t2fw_b200.functional_lfw import LFWFunction

    B, T, D, K, n_dec = 4, 1024, 64, 64, 6
    x, f, q, k, fk, s, _, _ = to_dev(lfw_inputs(B, T + n_dec, D, K, "sigmoid", 0.3, 91), torch.float16, cuda)
    with torch.no_grad():
        out_p, nxt = LFWFunction.apply(*[t[:, :T].contiguous() for t in (x, f, q, k, fk)], s)
    loop = LFWDecodeLoop(nxt, ring=2)
    outs = []
    for r in range(n_dec // 2):
        for i in range(2):
            t = T + 2 * r + i
            loop.x[i].copy_(x[:, t:t + 1]); loop.f[i].copy_(f[:, t:t + 1])
            loop.query[i].copy_(q[:, t:t + 1]); loop.key[i].copy_(k[:, t:t + 1]); loop.f_key[i].copy_(fk[:, t:t + 1])
        outs.append(loop.run_ring().clone())
    torch.cuda.synchronize()
    got = torch.cat([out_p] + [o[i] for o in outs for i in range(2)], dim=1)
    r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    assert max_rel_err(got, r_out) <= OUT_TOL[torch.float16]
    assert max_rel_err(loop.state, r_fin) <= OUT_TOL[torch.float16]
    assert loop.steps == n_dec


def test_decode_loop_replay_equals_eager_steps(cuda):
    from t2fw_b200.decode import LFWDecodeLoop, lfw_decode_step

    B, D, K, ring, trips = 64, 64, 64, 4, 3
    x, f, q, k, fk, s, _, _ = to_dev(lfw_inputs(B, ring, D, K, "sigmoid", 0.3, 92), torch.float16, cuda)
    loop = LFWDecodeLoop(s, ring=ring)
    for i in range(ring):
        loop.x[i].copy_(x[:, i:i + 1]); loop.f[i].copy_(f[:, i:i + 1])
        loop.query[i].copy_(q[:, i:i + 1]); loop.key[i].copy_(k[:, i:i + 1]); loop.f_key[i].copy_(fk[:, i:i + 1])
    a, b = s.clone(), torch.empty_like(s)
    o = torch.empty(B, 1, D, dtype=s.dtype, device=cuda)
    for trip in range(trips):
        got = loop.run_ring().clone()
        for i in range(ring):
            lfw_decode_step(x[:, i:i + 1].contiguous(), f[:, i:i + 1].contiguous(), q[:, i:i + 1].contiguous(),
                            k[:, i:i + 1].contiguous(), fk[:, i:i + 1].contiguous(), a, b, o)
            assert torch.equal(got[i], o), (trip, i)
            a, b = b, a
        assert torch.equal(loop.state, a)


def test_decode_step_rejects_in_place_state(cuda):
    from t2fw_b200.decode import lfw_decode_step

    x, f, q, k, fk, s, _, _ = to_dev(lfw_inputs(2, 1, 64, 64, "sigmoid", 0.3, 93), torch.float16, cuda)
    with pytest.raises(RuntimeError, match="alternate two buffers"):
        lfw_decode_step(x, f, q, k, fk, s, s, torch.empty_like(x))


def test_autograd_wrapper_under_graph_capture(cuda):
    """Forward + backward through LFWFunction.apply captured in a CUDA graph and replayed twice:
    bitwise equal to the eager result (the call neither synchronises nor depends on host state)."""
    from t2fw_b200.functional_lfw import LFWFunction

    x, f, q, k, fk, s, go, gs = to_dev(lfw_inputs(8, 256, 64, 64, "sigmoid", 0.3, 94), torch.float16, cuda)
    def run():
        # fresh leaves per run, so that autograd's bookkeeping for them belongs to the stream the
        # run is on (leaves made earlier on the default stream would make it synchronise with it)
        leaves = [t.detach().requires_grad_(True) for t in (x, f, q, k, fk, s)]
        out, nxt = LFWFunction.apply(*leaves)
        return [out, nxt] + list(torch.autograd.grad([out, nxt], leaves, [go, gs]))

    eager = [t.clone() for t in run()]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()                                    # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        static = run()
    for _ in range(2):
        for t in static:
            t.detach().fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        for a, b in zip(static, eager):
            assert torch.equal(a, b)
    r_out, _ = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    assert max_rel_err(static[0], r_out) <= OUT_TOL[torch.float16]
