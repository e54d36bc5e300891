"""Per-head GroupNorm of the WKV output plus the (r.k.r_k) v bonus, times the gate.

Mirror of the reference's `flashrwkv2/tmix/lnx_rkvres_xg/__init__.py:10-89`.
"""
from __future__ import annotations

from ..._ext import extension
from .._checks import check_io
from .pretrain import pretrain_tmix_lnx_rkvres_xg_bf16


def infer_tmix_lnx_rkvres_xg_forward_varlen(x, r, k, v, r_k, weight, bias, g, *, head_size: int = 64,
                                            batch_size: int = 1, max_seqlen: int | None = None):
    for name, tensor in (("x", x), ("r", r), ("k", k), ("v", v), ("r_k", r_k), ("weight", weight), ("bias", bias),
                         ("g", g)):
        check_io(name, tensor, x if name != "x" else None)
    if x.ndim != 2 or x.shape[0] <= 0 or x.shape[1] <= 0:
        raise ValueError("x must have packed shape [total_tokens,C]")
    if any(t.shape != x.shape for t in (r, k, v, g)):
        raise ValueError("r, k, v and g must match x's packed shape")
    if any(t.shape != (x.shape[1],) for t in (r_k, weight, bias)):
        raise ValueError("r_k, weight and bias must have shape [C]")
    if head_size not in (64, 128, 256) or x.shape[1] % head_size:
        raise ValueError("head_size must be 64, 128, or 256 and divide C")
    if batch_size <= 0 or (max_seqlen is not None and max_seqlen <= 0):
        raise ValueError("batch_size and max_seqlen must be positive")
    return extension().tmix_lnx_rkvres_xg_forward_varlen(x, r, k, v, r_k, weight, bias, g, int(head_size),
                                                         int(batch_size), 1 if max_seqlen is None else int(max_seqlen))


__all__ = ["infer_tmix_lnx_rkvres_xg_forward_varlen", "pretrain_tmix_lnx_rkvres_xg_bf16"]
