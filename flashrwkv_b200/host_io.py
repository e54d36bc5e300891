"""Decode from host buffers: a three-stream loop around `infer_recurrent_fp32io16_forward_varlen`.

A serving host holds the per-step token tensors (`r, decay_logits, k, v, a, b`) in pinned host memory and wants
the outputs back in host memory.  One decode step moves 6 x the token bytes to the device and 1 x back, which over
PCIe takes longer than the kernel itself, so the loop keeps the three engines busy at the same time:

    copy-in stream  : step i+1's six host -> device copies
    compute stream  : step i's kernel (the stream the metadata ticket was prepared on)
    copy-out stream : step i-1's device -> host copy

The state pool is updated in place in submission order (all kernels are on the compute stream); device staging
buffers and output buffers rotate over `depth` slots guarded by events.  Nothing here synchronises the host:
`drain()` makes the compute stream wait for the last copy-out so that a caller can time or order against it.
"""
from __future__ import annotations

import torch

from .tmix.wkv7 import infer_recurrent_fp32io16_forward_varlen


class HostDecodeLoop:
    def __init__(self, example_inputs, *, state_pool, cu_seqlens, state_indices, validated_metadata,
                 max_seqlen: int | None = 1, scale: float = 1.0, decay_bias=None, depth: int = 3):
        if depth < 2:
            raise ValueError("depth must be at least 2")
        if len(example_inputs) != 6:
            raise ValueError("six token tensors (r, decay_logits, k, v, a, b) are expected")
        for t in example_inputs:
            if t.device.type != "cpu" or not t.is_pinned():
                raise ValueError("token tensors must be pinned host tensors")
        dev = state_pool.device
        self._kw = dict(state_pool=state_pool, cu_seqlens=cu_seqlens, state_indices=state_indices,
                        validated_metadata=validated_metadata, max_seqlen=max_seqlen, scale=scale,
                        decay_bias=decay_bias)
        self._depth = depth
        self._compute = torch.cuda.current_stream(dev)
        self._copy_in = torch.cuda.Stream(dev)
        self._copy_out = torch.cuda.Stream(dev)
        # one device buffer [6, N, H, D] per slot: six separate host tensors are copied into its rows, a host
        # buffer of the same packed shape goes over in a single copy (one DMA descriptor instead of six)
        first = example_inputs[0]
        for t in example_inputs:
            if t.shape != first.shape or t.dtype != first.dtype:
                raise ValueError("the six token tensors must have one shape and dtype")
        self._packed = [torch.empty((6, *first.shape), dtype=first.dtype, device=dev) for _ in range(depth)]
        self._stage = [list(p.unbind(0)) for p in self._packed]
        self._outputs = [None] * depth
        self._loaded = [torch.cuda.Event() for _ in range(depth)]
        self._computed = [torch.cuda.Event() for _ in range(depth)]
        self._returned = [torch.cuda.Event() for _ in range(depth)]
        self._steps = 0

    def submit(self, host_inputs, host_output) -> None:
        """Queue one decode step: `host_inputs` in, `host_output` (pinned) out.

        `host_inputs` is either six pinned tensors `(r, decay_logits, k, v, a, b)` or one pinned tensor
        `[6, N, H, D]` holding them in that order (copied with a single transfer).
        """
        slot = self._steps % self._depth
        reused = self._steps >= self._depth
        stage = self._stage[slot]
        if reused:
            self._copy_in.wait_event(self._computed[slot])  # the kernel that read this staging slot has finished
        with torch.cuda.stream(self._copy_in):
            if isinstance(host_inputs, torch.Tensor):
                self._packed[slot].copy_(host_inputs, non_blocking=True)
            else:
                for d, s in zip(stage, host_inputs):
                    d.copy_(s, non_blocking=True)
            self._loaded[slot].record(self._copy_in)
        self._compute.wait_event(self._loaded[slot])
        if reused:
            # the output buffer of this slot goes back to the allocator below: its copy-out must be over first
            self._compute.wait_event(self._returned[slot])
        y = infer_recurrent_fp32io16_forward_varlen(*stage, **self._kw)
        self._outputs[slot] = y
        self._computed[slot].record(self._compute)
        self._copy_out.wait_event(self._computed[slot])
        with torch.cuda.stream(self._copy_out):
            host_output.copy_(y, non_blocking=True)
            self._returned[slot].record(self._copy_out)
        self._steps += 1

    def drain(self) -> None:
        """Order the compute stream after every copy queued so far (no host synchronisation)."""
        self._compute.wait_stream(self._copy_out)
        self._compute.wait_stream(self._copy_in)


__all__ = ["HostDecodeLoop"]
