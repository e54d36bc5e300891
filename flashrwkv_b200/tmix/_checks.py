"""Argument checks shared by the TMix operator wrappers (raise before any launch)."""
from __future__ import annotations

import torch

IO_DTYPES = (torch.float16, torch.bfloat16)


def check_io(name: str, tensor, ref=None) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if tensor.dtype not in IO_DTYPES:
        raise TypeError(f"{name} must have dtype torch.float16 or torch.bfloat16")
    if not tensor.is_cuda or not tensor.is_contiguous():
        raise ValueError(f"{name} must be CUDA and contiguous")
    if ref is not None:
        if tensor.dtype != ref.dtype:
            raise TypeError(f"{name} must have the same dtype as the first tensor")
        if tensor.device != ref.device:
            raise ValueError(f"{name} must share the first tensor's device")


def check_train_bf16(tensors: dict) -> None:
    """The training-side operators take contiguous CUDA bfloat16 tensors on one device (ValueError otherwise)."""
    first = None
    for name, tensor in tensors.items():
        if not isinstance(tensor, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if tensor.dtype != torch.bfloat16 or not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous CUDA bfloat16")
        if first is None:
            first = tensor
        elif tensor.device != first.device:
            raise ValueError(f"{name} must share {next(iter(tensors))}'s device")
