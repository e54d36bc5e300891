"""Block-level add / LayerNorm operators in front of the TMix group.

Mirror of the reference's `flashrwkv2/tmix/normalization/__init__.py:31-90` (names, keyword-only parameters,
returned tuples); fp16 as in the reference, bf16 in addition.  One kernel serves the four operators; statistics are
taken in fp32 from the rounded sum, the tensor the caller gets back.
"""
from __future__ import annotations

import torch

from ..._ext import extension
from .._checks import check_io


def _check_rows(tensor, name, reference=None) -> None:
    check_io(name, tensor, reference)
    if tensor.ndim != 2 or tensor.shape[0] <= 0 or tensor.shape[1] <= 0:
        raise ValueError(f"{name} must have packed shape [total_tokens,C]")
    if reference is not None and tensor.shape != reference.shape:
        raise ValueError(f"{name} must have the same shape as x")


def _check_affine(x, weight, bias) -> None:
    for name, t in (("weight", weight), ("bias", bias)):
        check_io(name, t, x)
        if t.shape != (x.shape[1],):
            raise ValueError(f"{name} must have shape [C]")


def _check_eps(eps) -> float:
    if not isinstance(eps, (int, float)) or isinstance(eps, bool) or not eps > 0 or eps != eps or eps == float("inf"):
        raise ValueError("eps must be positive")
    return float(eps)


def infer_tmix_layer_norm_forward_varlen(x, weight, bias, *, eps: float = 1.0e-5):
    _check_rows(x, "x")
    _check_affine(x, weight, bias)
    return extension().tmix_layer_norm_forward_varlen(x, weight, bias, _check_eps(eps))


def infer_tmix_add_layer_norm_forward_varlen(x, residual, weight, bias, *, eps: float = 1.0e-5,
                                             batch_size: int | None = None):
    """Returns `(x + residual, LayerNorm(x + residual))`."""
    _check_rows(x, "x")
    _check_rows(residual, "residual", x)
    _check_affine(x, weight, bias)
    if batch_size is not None and (not isinstance(batch_size, int) or isinstance(batch_size, bool) or batch_size <= 0
                                   or batch_size > x.shape[0]):
        raise ValueError("batch_size must be a positive integer no larger than total_tokens")
    return tuple(extension().tmix_add_layer_norm_forward_varlen(x, residual, weight, bias, _check_eps(eps),
                                                                -1 if batch_size is None else int(batch_size)))


def infer_tmix_add_last_layer_norm_forward_varlen(x, residual, weight, bias, *, eps: float = 1.0e-5):
    _check_rows(x, "x")
    _check_rows(residual, "residual", x)
    _check_affine(x, weight, bias)
    return extension().tmix_add_last_layer_norm_forward_varlen(x, residual, weight, bias, _check_eps(eps))


def infer_tmix_add_forward_varlen(x, residual):
    _check_rows(x, "x")
    _check_rows(residual, "residual", x)
    return extension().tmix_add_forward_varlen(x, residual)


__all__ = [
    "infer_tmix_layer_norm_forward_varlen",
    "infer_tmix_add_layer_norm_forward_varlen",
    "infer_tmix_add_last_layer_norm_forward_varlen",
    "infer_tmix_add_forward_varlen",
]
