"""WKV inputs from the projections: gated key, negative normalised key, gated normalised key.

Mirror of the reference's `flashrwkv2/tmix/kk_a_gate/__init__.py:10-72`.
"""
from __future__ import annotations

from ..._ext import extension
from .._checks import check_io


def infer_tmix_kk_a_gate_forward_varlen(k, k_k, a0, a12, k_a, *, head_size: int = 64, batch_size: int = 1,
                                        max_seqlen: int | None = None):
    for name, tensor in (("k", k), ("k_k", k_k), ("a0", a0), ("a12", a12), ("k_a", k_a)):
        check_io(name, tensor, k if name != "k" else None)
    if k.ndim != 2 or k.shape[0] <= 0 or k.shape[1] <= 0:
        raise ValueError("k must have packed shape [total_tokens,C]")
    if a12.shape != k.shape:
        raise ValueError("a12 must match k's packed shape")
    if any(t.shape != (k.shape[1],) for t in (k_k, a0, k_a)):
        raise ValueError("k_k, a0 and k_a must have shape [C]")
    if head_size not in (64, 128, 256) or k.shape[1] % head_size:
        raise ValueError("head_size must be 64, 128, or 256 and divide C")
    if batch_size <= 0 or (max_seqlen is not None and max_seqlen <= 0):
        raise ValueError("batch_size and max_seqlen must be positive")
    return extension().tmix_kk_a_gate_forward_varlen(k, k_k, a0, a12, k_a, int(head_size), int(batch_size),
                                                     1 if max_seqlen is None else int(max_seqlen))


__all__ = ["infer_tmix_kk_a_gate_forward_varlen"]
