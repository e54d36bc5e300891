"""Value residual gate: v + (v_first - v) * sigmoid(v0 + v12).

Mirror of the reference's `flashrwkv2/tmix/vres_gate/__init__.py:10-48`.
"""
from __future__ import annotations

import torch

from ..._ext import extension
from .._checks import check_io, check_train_bf16


def infer_tmix_vres_gate_forward_varlen(v, v_first, v0, v12):
    for name, tensor in (("v", v), ("v_first", v_first), ("v0", v0), ("v12", v12)):
        check_io(name, tensor, v if name != "v" else None)
    if v.ndim != 2 or v.shape[0] <= 0 or v.shape[1] <= 0:
        raise ValueError("v must have packed shape [total_tokens,C]")
    if v_first.shape != v.shape or v12.shape != v.shape:
        raise ValueError("v_first and v12 must match v's packed shape")
    if v0.shape != (v.shape[1],):
        raise ValueError("v0 must have shape [C]")
    return extension().tmix_vres_gate_forward_varlen(v, v_first, v0, v12)


class _VResGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, value, first_value, v0, v12):
        output = extension().pretrain_tmix_vres_gate_forward(value, first_value, v0, v12)
        ctx.save_for_backward(value, first_value, v0, v12)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        if grad_output is None:
            return None, None, None, None
        return tuple(extension().pretrain_tmix_vres_gate_backward(grad_output.contiguous(), *ctx.saved_tensors))


def pretrain_tmix_vres_gate_bf16(value, first_value, v0, v12):
    """Training-side value-residual gate on dense [B,T,C] bf16 tensors, with its backward (the gradient of v0 is a
    fixed-order fp32 sum over the rows).  Mirror of `flashrwkv2/tmix/vres_gate/__init__.py:36-71`."""
    check_train_bf16({"value": value, "first_value": first_value, "v0": v0, "v12": v12})
    if value.ndim != 3 or value.numel() == 0:
        raise ValueError("value must have shape [B,T,C]")
    if first_value.shape != value.shape or v12.shape != value.shape or v0.shape != (value.shape[-1],):
        raise ValueError("invalid v-residual gate shapes")
    return _VResGate.apply(value, first_value, v0, v12)


__all__ = ["infer_tmix_vres_gate_forward_varlen", "pretrain_tmix_vres_gate_bf16"]
