"""TMix token shift (six lerps with the previous token / shift state).

Mirror of the reference's `flashrwkv2/tmix/mix6/__init__.py:17-100`; fp16 as there, bf16 in addition.
"""
from __future__ import annotations

import torch

from ..._ext import extension
from .._checks import check_io, check_train_bf16
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


def infer_tmix_mix6_add_layer_norm_forward_varlen(x, residual, weight, bias, x_r, x_w, x_k, x_v, x_a, x_g, *,
                                                  shift_state_pool, cu_seqlens, state_indices,
                                                  max_seqlen: int | None = None, eps: float = 1.0e-5,
                                                  validated_metadata=None):
    """Add + LayerNorm + token shift: returns `(x + residual, six mixed tensors)` and stores the normalised last row of
    each sequence as its shift state (reference: `flashrwkv2/tmix/mix6/__init__.py:103-199`, which takes one row of
    4096 channels).  Batches of one-token sequences (`max_seqlen=1`) run as ONE kernel; anything else as add +
    LayerNorm followed by `infer_tmix_mix6_forward_varlen`.
    """
    from ..normalization import _check_affine, _check_eps, _check_rows, infer_tmix_add_layer_norm_forward_varlen

    _check_rows(x, "x")
    _check_rows(residual, "residual", x)
    _check_affine(x, weight, bias)
    mixes = (x_r, x_w, x_k, x_v, x_a, x_g)
    for name, t in zip(("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"), mixes):
        check_io(name, t, x)
        if t.shape != (x.shape[1],):
            raise ValueError("normalization and mix parameters must have shape [C]")
    if not isinstance(shift_state_pool, torch.Tensor):
        raise TypeError("shift_state_pool must be a torch.Tensor")
    if (shift_state_pool.dtype != x.dtype or not shift_state_pool.is_cuda or not shift_state_pool.is_contiguous()
            or shift_state_pool.ndim != 2 or shift_state_pool.shape[1] != x.shape[1]
            or shift_state_pool.device != x.device):
        raise ValueError("shift_state_pool must be contiguous CUDA [slots,C] of x's dtype on x's device")
    _check_metadata_inputs(cu_seqlens, state_indices)
    if max_seqlen is not None and (not isinstance(max_seqlen, int) or isinstance(max_seqlen, bool) or max_seqlen <= 0):
        raise ValueError("max_seqlen must be a positive integer")
    eps = _check_eps(eps)
    if max_seqlen == 1 and state_indices.numel() == x.shape[0]:
        return tuple(extension().tmix_mix6_add_layer_norm_forward_varlen(
            x, residual, weight, bias, shift_state_pool, *mixes, cu_seqlens, state_indices, 1, eps, validated_metadata))
    summed, normalized = infer_tmix_add_layer_norm_forward_varlen(x, residual, weight, bias, eps=eps)
    return (summed, *infer_tmix_mix6_forward_varlen(normalized, *mixes, shift_state_pool=shift_state_pool,
                                                    cu_seqlens=cu_seqlens, state_indices=state_indices,
                                                    max_seqlen=max_seqlen, validated_metadata=validated_metadata))


def infer_tmix_shift_project_forward_varlen(x, mixes, weights, *, shift_state_pool, cu_seqlens, state_indices,
                                            max_seqlen: int | None = None, validated_metadata=None,
                                            fuse_many_rows: bool = False):
    """Token shift fused into the projections that consume it (no counterpart in the reference, which runs
    `infer_tmix_mix6_forward_varlen` and then the projections).

    `outputs[j] = (x + (prev - x) * mixes[j]) @ weights[j]^T` for up to eight `(mix [C], weight [N_j,C])` pairs —
    e.g. r, k, v and the four rank-in projections of a TMix layer — and each sequence's last row goes to its
    shift-state slot.  With 1..8 rows this is one launch (plus the state update) and the interpolated rows never
    leave the chip.  With more rows the default is mix6 per distinct mix vector and the grouped GEMMs;
    `fuse_many_rows=True` does the interpolation inside the TMA-fed tensor-core GEMM instead, on its staged x tiles
    (four projections per launch).  That form is correct and tested but measured slower on B200 (the GEMM is bound
    by the fill of its shared-memory stages, and the extra pass over the x tile costs more than the six [M,C]
    tensors it saves: 114 against 90 us for r, k, v and the four rank-in products at M = 512, C = 2048).
    """
    from ..linear import _grouped

    mixes, weights = list(mixes), list(weights)
    if not mixes or len(mixes) != len(weights) or len(mixes) > 8:
        raise ValueError("1..8 mix vectors and as many weights are required")
    check_io("x", x, None)
    if x.ndim != 2 or x.shape[0] <= 0 or x.shape[1] <= 0:
        raise ValueError("x must have packed shape [total_tokens,C]")
    for name, group, shape_ok in (("mix", mixes, lambda t: t.shape == (x.shape[1],)),
                                  ("weight", weights, lambda t: t.ndim == 2 and t.shape[1] == x.shape[1])):
        for t in group:
            check_io(name, t, x)
            if not shape_ok(t):
                raise ValueError(f"every {name} must have shape " + ("[C]" if name == "mix" else "[N,C]"))
    if not isinstance(shift_state_pool, torch.Tensor):
        raise TypeError("shift_state_pool must be a torch.Tensor")
    if (shift_state_pool.dtype != x.dtype or not shift_state_pool.is_cuda or not shift_state_pool.is_contiguous()
            or shift_state_pool.ndim != 2 or shift_state_pool.shape[1] != x.shape[1]):
        raise ValueError("shift_state_pool must be contiguous CUDA [slots,C] of x's dtype")
    _check_metadata_inputs(cu_seqlens, state_indices)
    if max_seqlen is not None and (not isinstance(max_seqlen, int) or isinstance(max_seqlen, bool) or max_seqlen <= 0):
        raise ValueError("max_seqlen must be a positive integer")
    aligned = all(t.data_ptr() % 16 == 0 for t in (x, *mixes, *weights)) and all(w.shape[0] % 8 == 0 for w in weights)
    if x.shape[1] >= 256 and x.shape[1] % 8 == 0 and (x.shape[0] <= 8 or (fuse_many_rows and aligned)):
        # 1..8 rows: the small-row kernel; more (on request): the GEMM with the shift applied to its staged x tiles
        return tuple(extension().tmix_shift_project_varlen(
            x, shift_state_pool, mixes, weights, cu_seqlens, state_indices,
            -1 if max_seqlen is None else int(max_seqlen), validated_metadata))
    # many rows: the six-way kernel once (it also updates the shift states), then the GEMMs in groups of four
    distinct = []
    for m in mixes:
        if not any(m is d for d in distinct):
            distinct.append(m)
    if len(distinct) > 6:
        raise ValueError("with more than 8 rows at most six distinct mix vectors are supported")
    padded = distinct + [distinct[0]] * (6 - len(distinct))
    mixed = infer_tmix_mix6_forward_varlen(x, *padded, shift_state_pool=shift_state_pool, cu_seqlens=cu_seqlens,
                                           state_indices=state_indices, max_seqlen=max_seqlen,
                                           validated_metadata=validated_metadata)
    xs = [mixed[[m is d for d in distinct].index(True)] for m in mixes]
    outs = []
    for i in range(0, len(xs), 4):
        outs.extend(_grouped(xs[i:i + 4], weights[i:i + 4], ["none"] * len(xs[i:i + 4])))
    return tuple(outs)


class _PretrainMix6(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, x_r, x_w, x_k, x_v, x_a, x_g):
        output = extension().pretrain_tmix_mix6_forward(x, x_r, x_w, x_k, x_v, x_a, x_g)
        ctx.save_for_backward(x, x_r, x_w, x_k, x_v, x_a, x_g)
        return tuple(output)

    @staticmethod
    def backward(ctx, *grad_outputs):
        if all(g is None for g in grad_outputs):
            return (None,) * 7
        x = ctx.saved_tensors[0]
        zeros = None
        grads = []
        for g in grad_outputs:  # an output that took no part in the loss contributes a zero gradient
            if g is None:
                zeros = torch.zeros_like(x) if zeros is None else zeros
                g = zeros
            grads.append(g.contiguous())
        return tuple(extension().pretrain_tmix_mix6_backward(*grads, *ctx.saved_tensors))


def pretrain_tmix_mix6_bf16(x, x_r, x_w, x_k, x_v, x_a, x_g):
    """Training-side six-way token shift on a dense `[B,T,C]` bf16 tensor (the row before t = 0 is zero), with its
    backward.  Mirror of `flashrwkv2/tmix/mix6/__init__.py:222-297`; the gradients of the six mix vectors are
    fixed-order fp32 sums over the rows."""
    check_train_bf16({"x": x})
    if x.ndim != 3 or x.numel() == 0:
        raise ValueError("x must have shape [B,T,C]")
    for name, tensor in zip(("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"), (x_r, x_w, x_k, x_v, x_a, x_g)):
        if (not isinstance(tensor, torch.Tensor) or tensor.dtype != torch.bfloat16 or not tensor.is_cuda
                or not tensor.is_contiguous() or tensor.shape != (x.shape[-1],) or tensor.device != x.device):
            raise ValueError(f"{name} must be contiguous CUDA bfloat16 [C]")
    return _PretrainMix6.apply(x, x_r, x_w, x_k, x_v, x_a, x_g)


class _StatetuneMix6(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, initial_shift, x_r, x_w, x_k, x_v, x_a, x_g):
        outputs = tuple(extension().statetune_tmix_mix6_forward(x, initial_shift, x_r, x_w, x_k, x_v, x_a, x_g))
        ctx.save_for_backward(x, initial_shift, x_r, x_w, x_k, x_v, x_a, x_g)
        return outputs

    @staticmethod
    def backward(ctx, *grad_outputs):
        x, initial_shift = ctx.saved_tensors[:2]
        grads = []
        for g, like in zip(grad_outputs, (x,) * 6 + (initial_shift,)):
            grads.append(torch.zeros_like(like) if g is None else g.contiguous())
        return tuple(extension().statetune_tmix_mix6_backward(*grads, *ctx.saved_tensors))


def statetune_tmix_mix6_bf16(x, initial_shift, x_r, x_w, x_k, x_v, x_a, x_g):
    """Six-way token shift with a differentiable chunk-boundary shift state: the row before t = 0 is
    `initial_shift[b]`; returns the six mixed tensors and the final shift state `x[:, -1, :]`.  Mirror of
    `flashrwkv2/tmix/mix6/__init__.py:244-343` (there C must be even, here a multiple of 8)."""
    if not isinstance(x, torch.Tensor):
        raise TypeError("x must be a torch.Tensor")
    if x.dtype != torch.bfloat16:
        raise TypeError("x must have dtype torch.bfloat16")
    if not x.is_cuda or not x.is_contiguous():
        raise ValueError("x must be contiguous CUDA bfloat16 [B,T,C]")
    if x.ndim != 3 or any(size <= 0 for size in x.shape):
        raise ValueError("x must have non-empty shape [B,T,C]")
    if x.shape[2] % 8:
        raise ValueError("x channel dimension C must be divisible by 8")
    tensors = (initial_shift, x_r, x_w, x_k, x_v, x_a, x_g)
    names = ("initial_shift", "x_r", "x_w", "x_k", "x_v", "x_a", "x_g")
    shapes = ((x.shape[0], x.shape[2]),) + ((x.shape[2],),) * 6
    for name, tensor, shape in zip(names, tensors, shapes):
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.dtype != torch.bfloat16:
            raise TypeError(f"{name} must have dtype torch.bfloat16")
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous CUDA bfloat16")
        if tensor.shape != shape:
            raise ValueError(f"{name} must have shape {shape}")
        if tensor.device != x.device:
            raise ValueError(f"{name} must share x's device")
    return _StatetuneMix6.apply(x, *tensors)


__all__ = ["infer_tmix_mix6_forward_varlen", "infer_tmix_mix6_add_layer_norm_forward_varlen",
           "infer_tmix_shift_project_forward_varlen", "pretrain_tmix_mix6_bf16", "statetune_tmix_mix6_bf16"]
