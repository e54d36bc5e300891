"""Chunked (tensor-core) WKV7 forward operators.

`infer_chunk_bf16_forward_varlen` mirrors the reference operator of the same name
(`flashrwkv2/tmix/wkv7/chunk.py:17-125` there): packed bf16 tokens, a state pool
updated in place at `state_indices`, any positive `chunk_size` (rounded here to the
64-token tiles the tensor-core kernels use -- the result does not depend on it).
Beyond the reference contract the state pool may also be fp32 (the bf16 pool of the
reference is converted around the call; all arithmetic keeps an fp32 state).

`wkv7_chunk_forward` is the general form the other chunk operators are built on:
explicit chunk tables, optional per-chunk boundary states, fp16 or bf16 tokens.
"""
from __future__ import annotations

import math

import torch

from ..._ext import extension
from . import _check_metadata_inputs, prepare_recurrent_metadata

MAX_CHUNK = 64


def make_chunk_metadata(cu_seqlens: torch.Tensor, chunk_size: int = MAX_CHUNK):
    """Chunk tables for packed sequences: (sequence_chunk_offsets [B+1], starts [Cn], ends [Cn]), int32 on
    the device of `cu_seqlens`.  Reads `cu_seqlens` on the host once (request-batch preparation)."""
    if chunk_size <= 0 or chunk_size > MAX_CHUNK:
        raise ValueError(f"chunk_size must be in 1..{MAX_CHUNK}")
    offsets = cu_seqlens.detach().cpu().tolist()
    seq_offsets, starts, ends = [0], [], []
    for begin, end in zip(offsets[:-1], offsets[1:]):
        if end <= begin:
            raise ValueError("each sequence must be non-empty")
        for s in range(begin, end, chunk_size):
            starts.append(s)
            ends.append(min(s + chunk_size, end))
        seq_offsets.append(len(starts))
    dev = cu_seqlens.device
    mk = lambda x: torch.tensor(x, device=dev, dtype=torch.int32)  # noqa: E731
    return mk(seq_offsets), mk(starts), mk(ends)


def wkv7_chunk_forward(r, decay_logits, k, v, a, b, *, state, chunk_metadata, state_indices=None,
                       scale: float = 1.0, decay_bias=None, want_boundary: bool = False,
                       output_fp32: torch.Tensor | None = None, metadata_status=None,
                       state_dot_a: torch.Tensor | None = None, path: int = -1):
    """Chunked forward with an fp32 state `[slots,H,64,64]` updated in place.

    Returns `(output, boundary_or_None, error_flag)`; `boundary[c]` is the state at the start of chunk `c`.
    `path` picks the kernels: 0 = build + scan through a workspace (spreads the chunks of few sequences over the
    GPU), 1 = one fused kernel per (sequence, head) without a workspace, -1 = chosen from the batch.  A float32
    `state_dot_a` tensor shaped like `r`, if given, receives `S_{t-1}^T a_t` per token (fused kernel).
    """
    sco, cs, ce = chunk_metadata
    output = torch.empty_like(v)
    boundary = None
    if want_boundary:
        boundary = torch.empty((cs.numel(), r.shape[1], 64, 64), device=r.device, dtype=torch.float32)
    flag = extension().wkv7_chunk_forward(sco, cs, ce, state, r, decay_logits, k, v, a, b, output, float(scale),
                                          decay_bias, state_indices, boundary, output_fp32, metadata_status,
                                          state_dot_a, int(path))
    return output, boundary, flag


def infer_chunk_bf16_forward_varlen(r, decay_logits, k, v, a, b, *, state_pool, cu_seqlens, state_indices,
                                    chunk_size: int = 16, max_seqlen: int | None = None, scale: float = 1.0,
                                    decay_bias=None, validated_metadata=None, chunk_metadata=None,
                                    output_fp32: torch.Tensor | None = None) -> torch.Tensor:
    """RWKV-7 chunked forward on packed requests; updates `state_pool` in place at `state_indices`."""
    if not isinstance(chunk_size, int) or isinstance(chunk_size, bool):
        raise TypeError("chunk_size must be an integer")
    if chunk_size <= 0:
        raise ValueError("chunk_size must be positive")
    if not math.isfinite(float(scale)):
        raise ValueError("scale must be finite")
    tensors = {"r": r, "decay_logits": decay_logits, "k": k, "v": v, "a": a, "b": b}
    for name, tensor in tensors.items():
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.dtype != torch.bfloat16 or not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous CUDA bfloat16")
        if tensor.device != r.device:
            raise ValueError(f"{name} must share r's device")
        if tensor.shape != r.shape:
            raise ValueError(f"{name} must have the same shape as r")
    if r.ndim != 3 or r.shape[0] <= 0 or r.shape[1] <= 0 or r.shape[2] != 64:
        raise ValueError("packed chunk inputs must have shape [total_tokens,H,64]")
    if (not isinstance(state_pool, torch.Tensor) or state_pool.dtype not in (torch.bfloat16, torch.float32)
            or not state_pool.is_cuda or not state_pool.is_contiguous() or state_pool.ndim != 4
            or state_pool.shape[1:] != (r.shape[1], 64, 64) or state_pool.device != r.device):
        raise ValueError("state_pool must be contiguous CUDA bfloat16 (or float32) [slots,H,64,64]")
    _check_metadata_inputs(cu_seqlens, state_indices)
    if (cu_seqlens.dtype != torch.int32 or state_indices.dtype != torch.int32 or not cu_seqlens.is_cuda
            or not state_indices.is_cuda or not cu_seqlens.is_contiguous() or not state_indices.is_contiguous()
            or cu_seqlens.device != r.device or state_indices.device != r.device):
        raise ValueError("chunk metadata must be contiguous CUDA int32")
    if decay_bias is not None:
        if (decay_bias.dtype != torch.bfloat16 or not decay_bias.is_cuda or not decay_bias.is_contiguous()
                or decay_bias.device != r.device or decay_bias.shape not in {(r.shape[1], 64), (r.shape[1] * 64,)}):
            raise ValueError("decay_bias must be contiguous CUDA bfloat16 [H,64] or [H*64]")
    ticket = validated_metadata
    if ticket is None:
        ticket = prepare_recurrent_metadata(cu_seqlens, state_indices, total_tokens=r.shape[0],
                                            state_pool_size=state_pool.shape[0], max_seqlen=max_seqlen)
    else:
        ticket._check_compatible(cu_seqlens, state_indices, r.shape[0], state_pool.shape[0],
                                 -1 if max_seqlen is None else int(max_seqlen))
    if chunk_metadata is None:
        chunk_metadata = make_chunk_metadata(cu_seqlens, MAX_CHUNK)
    status = ticket._status()
    slots = ticket._state_indices_snapshot()
    if state_pool.dtype == torch.float32:
        out, _, _ = wkv7_chunk_forward(r, decay_logits, k, v, a, b, state=state_pool, chunk_metadata=chunk_metadata,
                                       state_indices=slots, scale=scale, decay_bias=decay_bias,
                                       output_fp32=output_fp32, metadata_status=status)
        return out
    # the reference's bf16 pool: selected slots are widened to fp32 for the call and rounded back afterwards
    index = slots.to(torch.int64)
    working = state_pool.index_select(0, index).float()
    out, _, _ = wkv7_chunk_forward(r, decay_logits, k, v, a, b, state=working, chunk_metadata=chunk_metadata,
                                   scale=scale, decay_bias=decay_bias, output_fp32=output_fp32,
                                   metadata_status=status)
    state_pool.index_copy_(0, index, working.to(torch.bfloat16))
    return out


__all__ = ["infer_chunk_bf16_forward_varlen", "wkv7_chunk_forward", "make_chunk_metadata"]
