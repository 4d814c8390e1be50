"""GPT-2-small with every attention layer replaced by a fast-weight layer (delta rule or decay rule).

The reference ships the two recurrences but no model around them; this is the caller its
tests imply: per head, keys are normalised the way tests/test_dfw.py:45-46 builds them
(softmax over the key dimension times a sigmoid write strength), the decay gate is a sigmoid
with the positive bias initialisation of tests/test_lfw.py:10-16, and heads are folded into the
batch dimension ([B, T, H*d] -> [B*H, T, d]) because every batch x head row is an independent
recurrence.  Everything except the recurrence call is stock PyTorch.

    model = GPT2FW(GPT2FWConfig(rule="dfw")).half().cuda()
    loss = model(token_ids, targets=token_ids)

Data parallelism over several GPUs is torch's DistributedDataParallel (NCCL gradient all-reduce);
the recurrences themselves need no communication.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .functional_dfw import DFWFunction
from .functional_fused import LFWFusedFunction, unfused_reference
from .functional_lfw import LFWFunction


@dataclass
class GPT2FWConfig:
    vocab_size: int = 50257
    n_positions: int = 1024
    d_model: int = 768
    n_head: int = 12
    n_layer: int = 12
    rule: str = "dfw"          # "dfw" (delta rule) or "lfw" (decay rule)
    gate_bias: float = 4.0     # decay gates start near sigmoid(4) = 0.98


class FastWeightAttention(nn.Module):
    """Causal token mixing by a fast-weight memory of shape [d_head, d_head] per head."""

    def __init__(self, cfg):
        super().__init__()
        assert cfg.d_model % cfg.n_head == 0
        self.h, self.d = cfg.n_head, cfg.d_model // cfg.n_head
        self.rule = cfg.rule
        n_proj = 3 if cfg.rule == "dfw" else 4          # q, k, v (+ key-side decay gate)
        self.qkv = nn.Linear(cfg.d_model, n_proj * cfg.d_model)
        if cfg.rule == "dfw":
            self.strength = nn.Linear(cfg.d_model, cfg.n_head)   # write strength per head
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)

    def _fold(self, t, B, T):
        # [B, T, H*d] -> [B*H, T, d], contiguous as the operators require
        return t.view(B, T, self.h, self.d).permute(0, 2, 1, 3).reshape(B * self.h, T, self.d)

    def forward(self, x):
        B, T, C = x.shape
        if self.rule == "lfw":
            # projection output = query | key | value | gate; the recurrence reads the heads in place
            # and applies the query scale and the gate activation itself (fused entry point); other
            # head sizes and dtypes take the same layer built from the plain operator
            qkvg = self.qkv(x)
            state = torch.zeros(B * self.h, self.d, self.d, dtype=x.dtype, device=x.device)
            if self.d == 64 and x.dtype in (torch.float16, torch.bfloat16) and x.is_cuda:
                out, _ = LFWFusedFunction.apply(qkvg, state, self.h)
            else:
                out, _ = unfused_reference(qkvg, state, self.h)
            return self.proj(out)
        parts = self.qkv(x).split(C, dim=-1)
        q, k, v = (self._fold(p, B, T) for p in parts[:3])
        state = torch.zeros(B * self.h, self.d, self.d, dtype=x.dtype, device=x.device)
        if True:
            beta = torch.sigmoid(self.strength(x))                       # [B, T, H]
            beta = beta.permute(0, 2, 1).reshape(B * self.h, T, 1)
            k = (torch.softmax(k.float(), dim=-1) * beta.float()).to(x.dtype)
            q = torch.softmax(q.float(), dim=-1).to(x.dtype)
            out, _ = DFWFunction.apply(q.contiguous(), k.contiguous(), v.contiguous(), state)
        out = out.view(B, self.h, T, self.d).permute(0, 2, 1, 3).reshape(B, T, C)
        return self.proj(out)


class Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.ln1 = nn.LayerNorm(cfg.d_model)
        self.attn = FastWeightAttention(cfg)
        self.ln2 = nn.LayerNorm(cfg.d_model)
        self.fc = nn.Linear(cfg.d_model, 4 * cfg.d_model)
        self.out = nn.Linear(4 * cfg.d_model, cfg.d_model)

    def forward(self, x):
        x = x + self.attn(self.ln1(x))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class GPT2FW(nn.Module):
    def __init__(self, cfg=None):
        super().__init__()
        self.cfg = cfg = cfg or GPT2FWConfig()
        # the table is padded to a multiple of 64 rows so that the output projection is an aligned
        # GEMM (ids and targets only ever use the first vocab_size rows)
        self.vocab_padded = (cfg.vocab_size + 63) // 64 * 64
        self.wte = nn.Embedding(self.vocab_padded, cfg.d_model)
        self.wpe = nn.Embedding(cfg.n_positions, cfg.d_model)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = nn.LayerNorm(cfg.d_model)
        self.apply(self._init)
        for blk in self.blocks:      # GPT-2's scaled init of the residual projections
            for lin in (blk.attn.proj, blk.out):
                nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))
            if cfg.rule == "lfw":    # decay gates start near 1 (tests/test_lfw.py:10-16)
                with torch.no_grad():
                    blk.attn.qkv.bias[3 * cfg.d_model:].fill_(cfg.gate_bias)

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)

    def n_params(self):
        return sum(p.numel() for p in self.parameters())

    def forward(self, ids, targets=None):
        B, T = ids.shape
        pos = torch.arange(T, device=ids.device)
        x = self.wte(ids) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)          # tied output embedding
        if targets is None:
            return logits
        return F.cross_entropy(logits.view(B * T, -1), targets.reshape(B * T)).float()
