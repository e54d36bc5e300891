"""Value residual gate: v + (v_first - v) * sigmoid(v0 + v12).

Mirror of the reference's `flashrwkv2/tmix/vres_gate/__init__.py:10-48`.
"""
from __future__ import annotations

from ..._ext import extension
from .._checks import check_io


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


__all__ = ["infer_tmix_vres_gate_forward_varlen"]
