"""Training-side a-gate: sigmoid(a0 + a12) on dense [B,T,C] bf16 tensors, with its backward.

Mirror of the reference's `flashrwkv2/tmix/a_gate/__init__.py:10-44`; the gradient of a0 is a fixed-order fp32 sum
over the B*T rows.
"""
from __future__ import annotations

import torch

from ..._ext import extension
from .._checks import check_train_bf16


def _check(a0, a12) -> None:
    check_train_bf16({"a12": a12, "a0": a0})
    if a0.ndim != 1 or a12.ndim != 3 or a0.shape != (a12.shape[-1],):
        raise ValueError("a0 must be [C] and a12 must be [B,T,C]")
    if any(size <= 0 for size in a12.shape):
        raise ValueError("a-gate inputs must be non-empty and share a device")


class _AGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a0, a12):
        output = extension().pretrain_tmix_a_gate_forward(a0, a12)
        ctx.save_for_backward(a0, a12)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        if grad_output is None:
            return None, None
        a0, a12 = ctx.saved_tensors
        gradients = extension().pretrain_tmix_a_gate_backward(grad_output.contiguous(), a0, a12)
        return gradients[0], gradients[1]


def pretrain_tmix_a_gate_bf16(a0, a12):
    _check(a0, a12)
    return _AGate.apply(a0, a12)


__all__ = ["pretrain_tmix_a_gate_bf16"]
