"""Training-side WKV7 operators with custom autograd: StateTune (non-zero fp32 initial state, caller-defined
chunks, gradient of the initial state) and dense BF16 pretraining (zero initial state).

Mirrors of the reference's `flashrwkv2/tmix/wkv7/statetune.py:79-236` and `pretrain.py:50-129`.  Forward = the
fused tensor-core chunk kernel, which also writes the chunk-start boundary states and `state_dot_a`.  Backward, on
the tensor cores as well: the adjoint of the state at every chunk boundary (the same fused kernel walking the
sequences backwards: the adjoint obeys a recurrence of the forward's form), then the token gradients of all
(chunk, head) pairs in parallel.  Head size 64.  Chunks handed to StateTune may hold at most 64 tokens each.
"""
from __future__ import annotations

import math

import torch

from ..._ext import extension
from .chunk import MAX_CHUNK

CHUNK_LEN = 16  # the reference's canonical pretraining chunk length: T must be a multiple of it


_last_flags = {}


def device_error_flags() -> dict:
    """Device error words (int32[1] tensors) of the most recent training forward and backward launched from this
    process.  A kernel whose bounded wait ran out has poisoned its outputs with NaN and left a non-zero value here;
    reading a flag synchronises, so the operators themselves never do."""
    return dict(_last_flags)


def check_device_error_flags() -> None:
    """Raise if the most recent training forward or backward reported a run-out wait (synchronises)."""
    for stage, flag in _last_flags.items():
        if int(flag.item()) != 0:
            raise RuntimeError(f"WKV7 training {stage}: a tensor-core completion wait ran out "
                               f"(device error flag {int(flag.item())}); its outputs are NaN")


def _forward_all(state, sco, cs, ce, r, w, k, v, a, b, scale):
    output = torch.empty_like(v)
    D = r.shape[2]
    boundary = torch.empty((cs.numel(), r.shape[1], D, D), device=r.device, dtype=torch.float32)
    state_dot_a = torch.empty(r.shape, device=r.device, dtype=torch.float32)
    if D != 64:  # head sizes 128 / 256: the plain-recurrence kernels (no tensor-core waits, hence no flag)
        extension().wkv7_train_wide_forward(sco, cs, ce, state, r, w, k, v, a, b, output, boundary, state_dot_a,
                                            float(scale))
        return output, boundary, state_dot_a, torch.zeros(1, dtype=torch.int32, device=r.device)
    flag = extension().wkv7_chunk_forward(sco, cs, ce, state, r, w, k, v, a, b, output, float(scale), None, None,
                                          boundary, None, None, state_dot_a, 1)
    _last_flags["forward"] = flag
    return output, boundary, state_dot_a, flag


def _backward_all(sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b, go, gf, scale):
    if r.shape[2] != 64:
        grads = extension().wkv7_train_wide_backward(sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b,
                                                     go, gf, float(scale))
        return grads, None
    *grads, flag = extension().wkv7_backward_chunked(sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b,
                                                     go, gf, float(scale))
    _last_flags["backward"] = flag
    return grads, flag


class _StateTune(torch.autograd.Function):
    @staticmethod
    def forward(ctx, initial_state, sco, cs, ce, r, w, k, v, a, b, scale):
        state = initial_state.detach().clone()  # the caller's initial state is never mutated
        output, boundary, state_dot_a, flag = _forward_all(state, sco, cs, ce, r.detach(), w.detach(), k.detach(),
                                                           v.detach(), a.detach(), b.detach(), scale)
        ctx.save_for_backward(sco, cs, ce, state, boundary, state_dot_a, r, w, k, v, a, b, flag)
        ctx.scale = scale
        ctx.mark_non_differentiable(boundary, state_dot_a)
        return output, state, boundary, state_dot_a

    @staticmethod
    def backward(ctx, grad_output, grad_final_state, _grad_boundary, _grad_sda):
        sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b, _flag = ctx.saved_tensors
        go = None if grad_output is None else grad_output.contiguous()
        gf = None if grad_final_state is None else grad_final_state.contiguous().float()
        (dr, dw, dk, dv, da, db, dS0), _ = _backward_all(sco, cs, ce, final_state, boundary, state_dot_a, r.detach(),
                                                         w.detach(), k.detach(), v.detach(), a.detach(), b.detach(),
                                                         go, gf, ctx.scale)
        return dS0, None, None, None, dr, dw, dk, dv, da, db, None


_validated_tables: list = []


def _validate_chunk_tables(sco, cs, ce, total_tokens: int) -> bool:
    """One device-to-host read for every property the kernels rely on: chunk bounds inside [0, N], chunks of a
    sequence contiguous and in order, offsets monotone from 0 to the chunk count.  A table that fails would drive
    out-of-range reads and writes on the device, so it is refused here.  Returns True when some chunk holds more
    than MAX_CHUNK tokens (the caller then splits those chunks; the kernels work on at most MAX_CHUNK)."""
    key = (sco, cs, ce)
    stamp = (sco._version, cs._version, ce._version, int(total_tokens))
    for entry in _validated_tables:
        if all(a is b for a, b in zip(entry[0], key)) and entry[1] == stamp:
            return entry[2]  # these very tensors, unmodified since, passed before (a training loop reuses its tables)
    cn = cs.numel()
    lens = ce - cs
    starts = torch.zeros(cn + 1, dtype=torch.bool, device=cs.device)
    starts[sco.clamp(0, cn).long()] = True
    code = ((lens > MAX_CHUNK).any().int() | (lens < 0).any().int() * 2 | (cs < 0).any().int() * 4
            | (ce > total_tokens).any().int() * 8 | (sco[0] != 0).int() * 16 | (sco[-1] != cn).int() * 32
            | (sco[1:] < sco[:-1]).any().int() * 64)
    if cn > 1:
        code = code | ((cs[1:] != ce[:-1]) & ~starts[1:cn]).any().int() * 128
    code = int(code.item())
    if code & (2 | 4 | 8):
        raise ValueError("chunk token bounds must satisfy 0 <= start <= end <= total_tokens")
    if code & (16 | 32 | 64):
        raise ValueError("sequence_chunk_offsets must rise from 0 to the number of chunks")
    if code & 128:
        raise ValueError("the chunks of a sequence must be contiguous and in token order")
    _validated_tables.append((key, stamp, bool(code & 1)))  # holds the tensors: their addresses cannot be recycled
    del _validated_tables[:-8]
    return bool(code & 1)


_refined_tables: list = []


def _refine_chunk_tables(sco, cs, ce):
    """Chunk tables whose chunks hold at most MAX_CHUNK tokens: every longer chunk of the caller is cut into pieces.
    Returns (sco, cs, ce, first) where first[c] is the index of the first piece of the caller's chunk c (the state at
    its start is the boundary the caller asked for).  Remembered per table identity and version."""
    key = (sco, cs, ce)
    stamp = (sco._version, cs._version, ce._version)
    for entry in _refined_tables:
        if all(a is b for a, b in zip(entry[0], key)) and entry[1] == stamp:
            return entry[2]
    h_sco, h_cs, h_ce = (t.cpu().tolist() for t in (sco, cs, ce))
    starts, ends, first, offsets = [], [], [], [0]
    for s in range(len(h_sco) - 1):
        for c in range(h_sco[s], h_sco[s + 1]):
            first.append(len(starts))
            a, b = h_cs[c], h_ce[c]
            if b <= a:
                starts.append(a)
                ends.append(b)
            while a < b:
                e = min(a + MAX_CHUNK, b)
                starts.append(a)
                ends.append(e)
                a = e
        offsets.append(len(starts))
    mk = lambda x, dt=torch.int32: torch.tensor(x, device=cs.device, dtype=dt)  # noqa: E731
    refined = (mk(offsets), mk(starts), mk(ends), mk(first, torch.int64))
    _refined_tables.append((key, stamp, refined))
    del _refined_tables[:-8]
    return refined


def _check_cuda_contiguous(tensor, name):
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not tensor.is_cuda or not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous CUDA")


def statetune_recurrent_fp32io16(initial_state, sequence_chunk_offsets, chunk_token_starts, chunk_token_ends, r,
                                 decay_logits, k, v, a, b, *, scale: float = 1.0):
    """StateTune forward with gradients for r, decay_logits, k, v, a, b and the initial state.

    Returns `(output [N,H,D], final_state [B,H,D,D], boundary [Cn,H,D,D], state_dot_a [N,H,D])`.
    """
    _check_cuda_contiguous(initial_state, "state")
    if initial_state.dtype != torch.float32:
        raise TypeError("state must be float32")
    if initial_state.ndim != 4 or initial_state.shape[0] <= 0 or initial_state.shape[1] <= 0:
        raise ValueError("state must have shape [B,H,D,D]")
    if initial_state.shape[2] != initial_state.shape[3] or initial_state.shape[2] not in (64, 128, 256):
        raise ValueError("state head size must be 64, 128, or 256")
    for name, tensor in (("r", r), ("decay_logits", decay_logits), ("k", k), ("v", v), ("a", a), ("b", b)):
        _check_cuda_contiguous(tensor, name)
        if tensor.device != initial_state.device:
            raise ValueError(f"{name} must share the state device")
        if tensor.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError(f"{name} must be float16 or bfloat16")
        if tensor.shape != r.shape or tensor.dtype != r.dtype:
            raise ValueError(f"{name} must match r shape and dtype")
    if r.ndim != 3 or r.shape[0] <= 0 or r.shape[1:] != initial_state.shape[1:3]:
        raise ValueError("token tensors must have shape [total_tokens,H,D]")
    for name, tensor in (("sequence_chunk_offsets", sequence_chunk_offsets), ("chunk_token_starts", chunk_token_starts),
                         ("chunk_token_ends", chunk_token_ends)):
        _check_cuda_contiguous(tensor, name)
        if tensor.dtype != torch.int32:
            raise TypeError(f"{name} must be int32")
        if tensor.device != initial_state.device:
            raise ValueError(f"{name} must share the state device")
    if sequence_chunk_offsets.ndim != 1:
        raise ValueError("sequence_chunk_offsets must be one-dimensional")
    if chunk_token_starts.ndim != 1 or chunk_token_ends.shape != chunk_token_starts.shape:
        raise ValueError("chunk token metadata must have matching shape [C]")
    if chunk_token_starts.numel() == 0:
        raise ValueError("at least one training chunk is required")
    if sequence_chunk_offsets.numel() != initial_state.shape[0] + 1:
        raise ValueError("sequence_chunk_offsets must have shape [B+1]")
    if not isinstance(scale, (int, float)) or not math.isfinite(float(scale)):
        raise ValueError("scale must be finite")
    if _validate_chunk_tables(sequence_chunk_offsets, chunk_token_starts, chunk_token_ends, r.shape[0]):
        # chunks longer than the kernels' 64 tokens: run on pieces, hand back the boundaries the caller's table names
        sco, cs, ce, first = _refine_chunk_tables(sequence_chunk_offsets, chunk_token_starts, chunk_token_ends)
        output, final_state, boundary, state_dot_a = _StateTune.apply(initial_state, sco, cs, ce, r, decay_logits, k, v,
                                                                      a, b, float(scale))
        return output, final_state, boundary.index_select(0, first), state_dot_a
    return _StateTune.apply(initial_state, sequence_chunk_offsets, chunk_token_starts, chunk_token_ends, r,
                            decay_logits, k, v, a, b, float(scale))


_dense_tables = {}


def _dense_chunk_tables(batch: int, tokens: int, device):
    key = (batch, tokens, str(device))
    if key not in _dense_tables:
        per = (tokens + MAX_CHUNK - 1) // MAX_CHUNK
        starts = [bi * tokens + c * MAX_CHUNK for bi in range(batch) for c in range(per)]
        ends = [min(s + MAX_CHUNK, (s // tokens + 1) * tokens) for s in starts]
        mk = lambda x: torch.tensor(x, device=device, dtype=torch.int32)  # noqa: E731
        _dense_tables[key] = (mk([bi * per for bi in range(batch + 1)]), mk(starts), mk(ends))
    return _dense_tables[key]


class _PretrainRecurrent(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, head_size):
        batch, tokens, channels = r.shape
        heads = channels // head_size
        tables = _dense_chunk_tables(batch, tokens, r.device)
        packed = [t.detach().view(batch * tokens, heads, head_size) for t in (r, w, k, v, a, b)]
        state = torch.zeros((batch, heads, head_size, head_size), device=r.device, dtype=torch.float32)  # S0 = 0
        output, boundary, state_dot_a, flag = _forward_all(state, *tables, *packed, 1.0)
        ctx.save_for_backward(*tables, state, boundary, state_dot_a, *packed, flag)
        ctx.shape = r.shape
        return output.view(r.shape)

    @staticmethod
    def backward(ctx, grad_output):
        sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b, _flag = ctx.saved_tensors
        go = grad_output.contiguous().view(r.shape)
        grads, _ = _backward_all(sco, cs, ce, final_state, boundary, state_dot_a, r, w, k, v, a, b, go, None, 1.0)
        return (*(g.view(ctx.shape) for g in grads[:6]), None)


def pretrain_recurrent_bf16(r, w, k, v, a, b, *, head_size: int = 64):
    """Dense `[B,T,C]` BF16 WKV7 with zero initial state and gradients for all six inputs (`w` is the raw decay
    input the retention transform is applied to)."""
    if head_size not in {64, 128, 256}:
        raise ValueError("head_size must be one of 64, 128, or 256")
    if not isinstance(r, torch.Tensor):
        raise TypeError("r must be a torch.Tensor")
    if r.ndim != 3 or min(r.shape) <= 0:
        raise ValueError("r must have shape [B,T,C] with nonzero dimensions")
    if r.dtype != torch.bfloat16:
        raise TypeError("r must be bfloat16")
    if not r.is_cuda or not r.is_contiguous():
        raise ValueError("r must be contiguous CUDA")
    for name, tensor in zip(("w", "k", "v", "a", "b"), (w, k, v, a, b)):
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.dtype != torch.bfloat16:
            raise TypeError(f"{name} must be bfloat16")
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous CUDA")
        if tensor.shape != r.shape:
            raise ValueError(f"{name} must match r shape")
        if tensor.device != r.device:
            raise ValueError(f"{name} must share the r device")
    if r.shape[2] % head_size != 0:
        raise ValueError("C must be divisible by head_size")
    if r.shape[1] % CHUNK_LEN != 0:
        raise ValueError("T must be divisible by the canonical chunk length 16")
    return _PretrainRecurrent.apply(r, w, k, v, a, b, head_size)


__all__ = ["statetune_recurrent_fp32io16", "pretrain_recurrent_bf16", "device_error_flags", "check_device_error_flags"]
