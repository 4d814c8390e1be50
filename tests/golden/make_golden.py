"""Generate golden input/output vectors by running the reference's own TorchScript functions.

Run in a container that has the reference checked out (it cannot travel to the GPU box):

    python tests/golden/make_golden.py /path/to/reference

It imports t2fw.torch from that checkout (t2fw/__init__.py is empty, so no CUDA build is
triggered), evaluates t2fw_torch / t2dfw_torch in float32 on CPU with autograd for the
gradients, and writes one .npz per case next to this script.  Inputs are stored with the
outputs so that the tests never depend on a random-number generator.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def gate_bias_init(shape):
    """Per-channel constant gates in (1/n, 1-1/n), the distribution the reference's unit tests
    use for f and f_key (tests/test_lfw.py:10-16,38,41)."""
    n = shape[-1]
    u = torch.rand(n) * (1 - 2.0 / n) + 1.0 / n if n > 2 else torch.full((n,), 0.5)
    return torch.sigmoid(torch.zeros(shape) - torch.log(1 / u - 1))


def lfw_inputs(B, T, D, K, gates, state_std, seed):
    torch.manual_seed(seed)
    x = torch.randn(B, T, D)
    q = torch.randn(B, T, K) / math.sqrt(K)
    k = torch.randn(B, T, K) / math.sqrt(K)
    if gates == "raw":            # literal N(0,1) f_key, two-sided with a sigmoid f
        fk = torch.randn(B, T, K)
        f = torch.sigmoid(torch.randn(B, T, D))
    elif gates == "raw_f1":       # f == 1, f_key ~ N(0,1): "gate taken from f_key"
        fk = torch.randn(B, T, K)
        f = torch.ones(B, T, D)
    elif gates == "sigmoid":      # time-varying gates in (0,1) on both sides
        fk = torch.sigmoid(torch.randn(B, T, K))
        f = torch.sigmoid(torch.randn(B, T, D))
    elif gates == "bias":         # the reference unit tests' constant per-channel gates
        fk = gate_bias_init((B, T, K))
        f = gate_bias_init((B, T, D))
    else:
        raise ValueError(gates)
    s = torch.randn(B, D, K) * state_std
    go = torch.randn(B, T, D)
    gs = torch.randn(B, D, K)
    return x, f, q, k, fk, s, go, gs


def dfw_inputs(B, T, D, M, keys, state_std, seed):
    torch.manual_seed(seed)
    v = torch.randn(B, T, D)
    q = torch.randn(B, T, M)
    k = torch.randn(B, T, M)
    if keys == "softmax":         # tests/test_dfw.py:45-46
        k = torch.softmax(k, dim=-1) * torch.sigmoid(k.mean(dim=-1, keepdim=True))
    elif keys == "scaled":        # N(0,1)/sqrt(M): |k|^2 ~ 1
        q = q / math.sqrt(M)
        k = k / math.sqrt(M)
    else:
        raise ValueError(keys)
    s = torch.randn(B, D, M) * state_std
    go = torch.randn(B, T, D)
    gs = torch.randn(B, D, M)
    return q, k, v, s, go, gs


LFW_CASES = [
    # name, B, T, D, K, gates, state_std, seed
    ("lfw_config1_raw", 2, 64, 64, 64, "raw", 0.1, 0),
    ("lfw_config1_rawf1", 2, 64, 64, 64, "raw_f1", 0.1, 1),
    ("lfw_config1_sigmoid", 2, 64, 64, 64, "sigmoid", 0.1, 2),
    ("lfw_tiny", 1, 1, 1, 1, "sigmoid", 1.0, 3),
    ("lfw_odd", 3, 37, 33, 17, "bias", 1.0, 4),
    ("lfw_t129", 2, 129, 32, 16, "bias", 1.0, 5),
    ("lfw_wide", 1, 20, 96, 48, "raw", 1.0, 6),
]

DFW_CASES = [
    ("dfw_config1_scaled", 2, 64, 64, 64, "scaled", 0.1, 10),
    ("dfw_config1_softmax", 2, 64, 64, 64, "softmax", 1.0, 11),
    ("dfw_tiny", 1, 1, 1, 1, "softmax", 1.0, 12),
    ("dfw_odd", 3, 37, 33, 17, "softmax", 1.0, 13),
    ("dfw_t129", 2, 129, 32, 16, "softmax", 1.0, 14),
]


def main(ref_root):
    sys.path.insert(0, ref_root)
    from t2fw.torch import t2fw_torch, t2dfw_torch, t2dfw_torch_bw  # the reference itself

    for name, B, T, D, K, gates, sstd, seed in LFW_CASES:
        x, f, q, k, fk, s, go, gs = lfw_inputs(B, T, D, K, gates, sstd, seed)
        leaves = [t.clone().requires_grad_(True) for t in (x, f, q, k, fk, s)]
        out, fin = t2fw_torch(*leaves)
        grads = torch.autograd.grad([out, fin], leaves, [go, gs])
        np.savez(os.path.join(HERE, name + ".npz"),
                 x=x.numpy(), f=f.numpy(), q=q.numpy(), k=k.numpy(), f_key=fk.numpy(),
                 state=s.numpy(), grad_out=go.numpy(), grad_state=gs.numpy(),
                 out=out.detach().numpy(), final_state=fin.detach().numpy(),
                 d_x=grads[0].numpy(), d_f=grads[1].numpy(), d_q=grads[2].numpy(),
                 d_k=grads[3].numpy(), d_f_key=grads[4].numpy(), d_state=grads[5].numpy())
        print("wrote", name)

    for name, B, T, D, M, keys, sstd, seed in DFW_CASES:
        q, k, v, s, go, gs = dfw_inputs(B, T, D, M, keys, sstd, seed)
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, s)]
        out, fin = t2dfw_torch(*leaves)
        grads = torch.autograd.grad([out, fin], leaves, [go, gs])
        # the reference's hand-written backward must agree with its own autograd
        hb = t2dfw_torch_bw(go, gs, q, k, v, s, fin.detach())
        for a, b in zip(hb, grads):
            assert torch.allclose(a, b, atol=1e-3, rtol=1e-3), name
        np.savez(os.path.join(HERE, name + ".npz"),
                 q=q.numpy(), k=k.numpy(), v=v.numpy(), state=s.numpy(),
                 grad_out=go.numpy(), grad_state=gs.numpy(),
                 out=out.detach().numpy(), final_state=fin.detach().numpy(),
                 d_q=grads[0].numpy(), d_k=grads[1].numpy(), d_v=grads[2].numpy(),
                 d_state=grads[3].numpy())
        print("wrote", name)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])
