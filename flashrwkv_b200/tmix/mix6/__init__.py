"""TMix token shift (six lerps with the previous token / shift state).

Mirror of the reference's `flashrwkv2/tmix/mix6/__init__.py:17-100`; fp16 as there, bf16 in addition.
"""
from __future__ import annotations

import torch

from ..._ext import extension
from .._checks import check_io
from ..wkv7 import _check_metadata_inputs


def infer_tmix_mix6_forward_varlen(x, x_r, x_w, x_k, x_v, x_a, x_g, *, shift_state_pool, cu_seqlens, state_indices,
                                   max_seqlen: int | None = None, validated_metadata=None):
    """Returns the six mixed `[N,C]` tensors and moves each sequence's last row into its shift-state slot."""
    names = ("x", "x_r", "x_w", "x_k", "x_v", "x_a", "x_g")
    tensors = (x, x_r, x_w, x_k, x_v, x_a, x_g)
    for name, tensor in zip(names, tensors):
        check_io(name, tensor, x if name != "x" else None)
    if x.ndim != 2 or x.shape[0] <= 0 or x.shape[1] <= 0:
        raise ValueError("x must have packed shape [total_tokens,C]")
    if any(t.shape != (x.shape[1],) for t in tensors[1:]):
        raise ValueError("all mix6 coefficients must have shape [C]")
    if not isinstance(shift_state_pool, torch.Tensor):
        raise TypeError("shift_state_pool must be a torch.Tensor")
    if (shift_state_pool.dtype != x.dtype or not shift_state_pool.is_cuda or not shift_state_pool.is_contiguous()
            or shift_state_pool.ndim != 2 or shift_state_pool.shape[1] != x.shape[1]):
        raise ValueError("shift_state_pool must be contiguous CUDA [slots,C] of x's dtype")
    if shift_state_pool.device != x.device:
        raise ValueError("shift_state_pool must share x's device")
    _check_metadata_inputs(cu_seqlens, state_indices)
    if max_seqlen is not None and (not isinstance(max_seqlen, int) or isinstance(max_seqlen, bool) or max_seqlen <= 0):
        raise ValueError("max_seqlen must be a positive integer")
    return tuple(extension().tmix_mix6_forward_varlen(
        x, shift_state_pool, x_r, x_w, x_k, x_v, x_a, x_g, cu_seqlens, state_indices,
        -1 if max_seqlen is None else int(max_seqlen), validated_metadata))


__all__ = ["infer_tmix_mix6_forward_varlen"]
