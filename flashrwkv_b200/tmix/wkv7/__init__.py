"""WKV7 recurrent inference operators.

Mirror of the reference's `flashrwkv2/tmix/wkv7/__init__.py` (public functions
at :180-277 there): same names, keyword-only parameters, validation order and
exception types; the native call goes to this package's `_C` module.
"""
from __future__ import annotations

import torch

from ..._ext import extension

_TOKEN_NAMES = ("r", "decay_logits", "k", "v", "a", "b")


def _validate_packed_inputs(*tensors):
    for name, tensor in zip(_TOKEN_NAMES, tensors):
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.ndim != 3:
            raise ValueError(f"{name} must have packed shape [total_tokens,H,D]")
        if not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    return tensors


def _validate_state(state) -> None:
    if not isinstance(state, torch.Tensor):
        raise TypeError("state_pool must be a torch.Tensor")
    if not state.is_contiguous():
        raise ValueError("state_pool must be contiguous")
    if state.dtype != torch.float32:
        raise TypeError("state_pool must have dtype float32")


def _check_metadata_inputs(cu_seqlens, state_indices) -> None:
    if not isinstance(cu_seqlens, torch.Tensor):
        raise TypeError("cu_seqlens must be a torch.Tensor")
    if cu_seqlens.ndim != 1:
        raise ValueError("cu_seqlens must be one-dimensional")
    if not isinstance(state_indices, torch.Tensor):
        raise TypeError("state_indices must be a torch.Tensor")


def prepare_recurrent_metadata(cu_seqlens, state_indices, *, total_tokens: int, state_pool_size: int,
                               max_seqlen: int | None = None):
    """Validate packed metadata on the device and return a reusable ticket.

    The ticket holds a snapshot of both tensors and a device status word; it can be
    passed as ``validated_metadata`` to any operator taking the same metadata on the
    same stream, which then launches without any host synchronisation.
    """
    _check_metadata_inputs(cu_seqlens, state_indices)
    return extension().prepare_recurrent_metadata(
        cu_seqlens, state_indices, total_tokens, state_pool_size,
        -1 if max_seqlen is None else int(max_seqlen))


def infer_recurrent_fp32io16_forward_varlen(r, decay_logits, k, v, a, b, *, state_pool, cu_seqlens,
                                            state_indices, scale: float = 1.0, decay_bias=None,
                                            max_seqlen: int | None = None, validated_metadata=None,
                                            output_fp32: torch.Tensor | None = None) -> torch.Tensor:
    """Packed raw-decay RWKV-7 recurrence, in place on the fp32 ``state_pool``.

    ``r, decay_logits, k, v, a, b`` are matching fp16/bf16 ``[N,H,D]`` tensors,
    ``state_pool`` is fp32 ``[slots,H,D,D]``.  Returns the output shaped like ``v``.
    ``output_fp32`` (an extension over the reference signature) optionally receives
    the outputs before rounding to the io dtype.
    """
    packed = _validate_packed_inputs(r, decay_logits, k, v, a, b)
    _validate_state(state_pool)
    _check_metadata_inputs(cu_seqlens, state_indices)
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_recurrent_metadata(cu_seqlens, state_indices, total_tokens=r.shape[0],
                                            state_pool_size=state_pool.shape[0], max_seqlen=max_seqlen)
    output = torch.empty_like(packed[3])
    extension().recurrent_fp32_from_decay_logits(
        cu_seqlens, state_indices, state_pool, *packed, output, float(scale), decay_bias, ticket,
        -1 if max_seqlen is None else int(max_seqlen), output_fp32)
    return output


__all__ = ["infer_recurrent_fp32io16_forward_varlen", "prepare_recurrent_metadata"]

from .chunk import infer_chunk_bf16_forward_varlen, make_chunk_metadata, wkv7_chunk_forward  # noqa: E402

__all__ += ["infer_chunk_bf16_forward_varlen", "wkv7_chunk_forward", "make_chunk_metadata"]

from .training import pretrain_recurrent_bf16, statetune_recurrent_fp32io16  # noqa: E402

__all__ += ["pretrain_recurrent_bf16", "statetune_recurrent_fp32io16"]
