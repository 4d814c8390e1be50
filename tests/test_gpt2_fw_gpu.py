"""The attention replacement of t2fw_b200/gpt2_fw.py against the same layer computed with the
step-by-step CPU port of the reference's recurrences (oracle/torch_port.py), and a smoke run of
the whole model."""
import copy

import pytest
import torch

from helpers import max_rel_err
from oracle import torch_port
from t2fw_b200.functional_fused import GATE_FLOOR

pytestmark = pytest.mark.gpu


def reference_layer(layer, x):
    """FastWeightAttention.forward with the recurrence done by the oracle's per-step loop (CPU, fp32)."""
    B, T, C = x.shape
    parts = layer.qkv(x).split(C, dim=-1)
    q, k, v = (layer._fold(p, B, T) for p in parts[:3])
    state = torch.zeros(B * layer.h, layer.d, layer.d)
    if layer.rule == "dfw":
        beta = torch.sigmoid(layer.strength(x)).permute(0, 2, 1).reshape(B * layer.h, T, 1)
        k = torch.softmax(k, dim=-1) * beta
        q = torch.softmax(q, dim=-1)
        out, _ = torch_port.dfw_loop(q, k, v, state)
    else:
        # the layer's gate is max(sigmoid(.), 1/8) (t2fw_b200/functional_fused.py)
        gate = torch.sigmoid(layer._fold(parts[3], B, T)).clamp_min(GATE_FLOOR)
        out, _ = torch_port.lfw_loop(v, torch.ones_like(v), q * layer.d ** -0.5, k, gate, state)
    out = out.view(B, layer.h, T, layer.d).permute(0, 2, 1, 3).reshape(B, T, C)
    return layer.proj(out)


@pytest.mark.parametrize("rule", ["dfw", "lfw"])
def test_attention_replacement_matches_cpu_port(cuda, rule):
    from t2fw_b200.gpt2_fw import FastWeightAttention, GPT2FWConfig

    torch.manual_seed(5)
    cfg = GPT2FWConfig(d_model=64, n_head=2, n_layer=1, rule=rule)
    cpu_layer = FastWeightAttention(cfg)
    gpu_layer = copy.deepcopy(cpu_layer).to(cuda)
    x = torch.randn(2, 70, 64)
    xc = x.clone().requires_grad_(True)
    xg = x.to(cuda).requires_grad_(True)
    yc = reference_layer(cpu_layer, xc)
    yg = gpu_layer(xg)
    w = torch.randn_like(yc)
    yc.backward(w)
    yg.backward(w.to(cuda))
    assert max_rel_err(yg, yc) <= 2e-4
    assert max_rel_err(xg.grad, xc.grad) <= 5e-4
    for (n, pc), pg in zip(cpu_layer.named_parameters(), gpu_layer.parameters()):
        assert max_rel_err(pg.grad, pc.grad) <= 1e-3, n


@pytest.mark.parametrize("rule", ["dfw", "lfw"])
def test_small_model_trains_in_fp16(cuda, rule):
    """Two layers, d_head = 64 (the chunked tensor-core kernels), a few AdamW steps on one batch:
    the loss is finite and goes down."""
    from t2fw_b200.gpt2_fw import GPT2FW, GPT2FWConfig

    torch.manual_seed(6)
    cfg = GPT2FWConfig(vocab_size=512, n_positions=256, d_model=128, n_head=2, n_layer=2, rule=rule)
    model = GPT2FW(cfg).half().to(cuda)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, eps=1e-4)
    ids = torch.randint(0, 512, (4, 257), device=cuda)
    losses = []
    for _ in range(8):
        loss = model(ids[:, :-1], targets=ids[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(loss.detach()))
    assert all(l == l and l < 1e4 for l in losses), losses
    assert losses[-1] < losses[0], losses
