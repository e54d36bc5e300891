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


# ---- fp16 state pool (reference: flashrwkv2/tmix/wkv7/__init__.py:41-140,280-339) ---------------------------------
def _validate_fp16_state(state) -> None:
    if not isinstance(state, torch.Tensor):
        raise TypeError("state_pool must be a torch.Tensor")
    if not state.is_contiguous():
        raise ValueError("state_pool must be contiguous")
    if state.dtype != torch.float16:
        raise TypeError("FP16-state state_pool must have dtype float16")


def _validate_elapsed(elapsed, name: str) -> None:
    if not isinstance(elapsed, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if elapsed.dtype != torch.int32:
        raise TypeError(f"{name} must have dtype torch.int32")
    if not elapsed.is_cuda or not elapsed.is_contiguous():
        raise ValueError(f"{name} must be contiguous CUDA int32")


def infer_recurrent_add_vec_forward_varlen(x, vec):
    """`x [total_tokens,C] + vec [C]` with one rounding (the recurrence's pre-add-vector helper).  Mirror of
    `flashrwkv2/tmix/wkv7/__init__.py:133-151`: fp16 as there, bf16 in addition."""
    for name, tensor in (("x", x), ("vec", vec)):
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.dtype not in (torch.float16, torch.bfloat16) or tensor.dtype != x.dtype:
            raise TypeError(f"{name} must have dtype torch.float16 (or both torch.bfloat16)")
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous CUDA float16")
        if tensor.device != x.device:
            raise ValueError(f"{name} must share x's device")
    if x.ndim != 2 or x.shape[0] <= 0 or x.shape[1] <= 0 or x.shape[1] % 2:
        raise ValueError("x must have packed shape [total_tokens,C] with even C")
    if vec.shape != (x.shape[1],):
        raise ValueError("vec must have shape [C]")
    return extension().recurrent_add_vec_forward_varlen(x, vec)


def infer_recurrent_fp16_advance_i32(elapsed_state, amount: int) -> None:
    """Add ``amount`` to every elapsed (dither phase) counter, in place."""
    _validate_elapsed(elapsed_state, "elapsed_state")
    if elapsed_state.numel() == 0:
        raise ValueError("elapsed_state must be non-empty")
    if not isinstance(amount, int) or isinstance(amount, bool):
        raise TypeError("amount must be an int")
    extension().recurrent_fp16_advance_i32(elapsed_state, amount)


def infer_recurrent_fp16_advance_i32_varlen(elapsed_state_pool, cu_seqlens, state_indices, *, total_tokens: int,
                                            validated_metadata=None) -> None:
    """Advance the counters of the selected slots by their sequences' packed lengths, in place."""
    if not isinstance(elapsed_state_pool, torch.Tensor):
        raise TypeError("elapsed_state_pool must be a torch.Tensor")
    if (elapsed_state_pool.dtype != torch.int32 or not elapsed_state_pool.is_cuda
            or not elapsed_state_pool.is_contiguous() or elapsed_state_pool.ndim != 1
            or elapsed_state_pool.numel() == 0):
        raise ValueError("elapsed_state_pool must be non-empty contiguous CUDA int32")
    _check_metadata_inputs(cu_seqlens, state_indices)
    for name, t in (("cu_seqlens", cu_seqlens), ("state_indices", state_indices)):
        if t.dtype != torch.int32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous CUDA int32")
        if t.device != elapsed_state_pool.device:
            raise ValueError("elapsed metadata tensors must share a CUDA device")
    if state_indices.ndim != 1 or cu_seqlens.numel() != state_indices.numel() + 1:
        raise ValueError("cu_seqlens must have shape [B+1] and state_indices shape [B]")
    if not isinstance(total_tokens, int) or isinstance(total_tokens, bool) or total_tokens <= 0:
        raise ValueError("total_tokens must be a positive integer")
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_recurrent_metadata(cu_seqlens, state_indices, total_tokens=total_tokens,
                                            state_pool_size=elapsed_state_pool.shape[0])
    extension().recurrent_fp16_advance_i32_varlen(cu_seqlens, state_indices, elapsed_state_pool, total_tokens, ticket)


def infer_recurrent_fp16_forward_varlen(r, decay_logits, k, v, a, b, *, state_pool, elapsed_state_pool, cu_seqlens,
                                        state_indices, scale: float = 1.0, decay_bias=None,
                                        max_seqlen: int | None = None, validated_metadata=None) -> torch.Tensor:
    """Packed RWKV-7 recurrence on an fp16 ``state_pool [slots,H,D,D]`` (D = 64, 128 or 256), updated in place.

    The retention enters as a rounded fp16 increment with a deterministic dither whose phase comes from the int32
    ``elapsed_state_pool [slots]`` (read, never advanced here: see the two ``advance`` operators).  Returns the
    output shaped like ``v``.
    """
    packed = _validate_packed_inputs(r, decay_logits, k, v, a, b)
    _validate_fp16_state(state_pool)
    _validate_elapsed(elapsed_state_pool, "elapsed_state_pool")
    if elapsed_state_pool.device != state_pool.device:
        raise ValueError("elapsed_state_pool must share state_pool's device")
    if elapsed_state_pool.ndim != 1 or elapsed_state_pool.shape[0] != state_pool.shape[0]:
        raise ValueError("elapsed_state_pool must have shape [state_pool_slots]")
    _check_metadata_inputs(cu_seqlens, state_indices)
    if max_seqlen is None:
        launch_max_seqlen = -1
    else:
        if not isinstance(max_seqlen, int) or isinstance(max_seqlen, bool) or max_seqlen <= 0:
            raise ValueError("max_seqlen must be a positive integer")
        launch_max_seqlen = int(max_seqlen)
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_recurrent_metadata(cu_seqlens, state_indices, total_tokens=r.shape[0],
                                            state_pool_size=state_pool.shape[0],
                                            max_seqlen=None if launch_max_seqlen < 0 else launch_max_seqlen)
    output = torch.empty_like(packed[3])
    extension().recurrent_fp16_from_decay_logits(
        cu_seqlens, state_indices, elapsed_state_pool, state_pool, *packed, output, float(scale), decay_bias, ticket,
        launch_max_seqlen)
    return output


__all__ = ["infer_recurrent_fp32io16_forward_varlen", "prepare_recurrent_metadata",
           "infer_recurrent_fp16_forward_varlen", "infer_recurrent_fp16_advance_i32",
           "infer_recurrent_fp16_advance_i32_varlen", "infer_recurrent_add_vec_forward_varlen"]

from .chunk import infer_chunk_bf16_forward_varlen, make_chunk_metadata, wkv7_chunk_forward  # noqa: E402

__all__ += ["infer_chunk_bf16_forward_varlen", "wkv7_chunk_forward", "make_chunk_metadata"]

from .training import pretrain_recurrent_bf16, statetune_recurrent_fp32io16  # noqa: E402

__all__ += ["pretrain_recurrent_bf16", "statetune_recurrent_fp32io16"]
