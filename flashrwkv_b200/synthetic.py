"""Seeded synthetic inputs with the value distributions of the benchmark configurations.

r, v ~ N(0,1); k ~ N(0,1) L2-normalised per head; the per-step log-decay is
-exp(u) with u ~ U(-4,-0.5), handed to the operators as the raw decay logit
that reproduces it (the operators apply w = exp(-exp(-0.5)*sigmoid(logit)), so
logit = log(p/(1-p)) with p = exp(u+0.5)); kk ~ N(0,1) L2-normalised, a = -kk,
b = kk*sigmoid(N(0,1)).  Everything is generated in fp32 on the CPU generator,
so a seed gives the same tensors on every machine, then cast once.
"""
from __future__ import annotations

import torch


def wkv7_inputs(total_tokens: int, num_heads: int, head_size: int, *, seed: int,
                dtype: torch.dtype = torch.bfloat16, device="cpu"):
    """Return (r, decay_logits, k, v, a, b), each [total_tokens, H, D] of ``dtype``."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    shape = (total_tokens, num_heads, head_size)
    r = torch.randn(shape, generator=g)
    k = torch.nn.functional.normalize(torch.randn(shape, generator=g), dim=-1)
    v = torch.randn(shape, generator=g)
    u = torch.rand(shape, generator=g) * 3.5 - 4.0
    p = torch.exp(u + 0.5).clamp_(max=1.0 - 1e-6)
    decay_logits = torch.log(p) - torch.log1p(-p)
    kk = torch.nn.functional.normalize(torch.randn(shape, generator=g), dim=-1)
    a = -kk
    b = kk * torch.sigmoid(torch.randn(shape, generator=g))
    return tuple(t.to(dtype).to(device) for t in (r, decay_logits, k, v, a, b))


def state_pool(slots: int, num_heads: int, head_size: int, *, seed: int, std: float = 0.1,
               device="cpu") -> torch.Tensor:
    """fp32 state pool [slots, H, D, D] ~ N(0, std)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return (torch.randn((slots, num_heads, head_size, head_size), generator=g) * std).to(device)


def equal_length_metadata(batch: int, seqlen: int, device="cpu"):
    """cu_seqlens = [0, T, 2T, ...] and state_indices = arange(batch), int32."""
    cu = torch.arange(batch + 1, dtype=torch.int32) * seqlen
    idx = torch.arange(batch, dtype=torch.int32)
    return cu.to(device), idx.to(device)
