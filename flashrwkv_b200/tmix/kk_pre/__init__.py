"""Training-side key preparation: per-head normalised key direction and the learning-rate-scaled key.

    kk = normalize(key * key_scale) per head (eps 1e-12)
    returns (key * (1 + (learning_rate - 1) * learning_rate_scale), -kk, kk * learning_rate)

Mirror of the reference's `flashrwkv2/tmix/kk_pre/__init__.py:10-71`.
"""
from __future__ import annotations

import torch

from ..._ext import extension
from .._checks import check_train_bf16


def _check_inputs(key, key_scale, learning_rate, learning_rate_scale, head_size) -> None:
    if head_size not in {64, 128, 256}:
        raise ValueError("head_size must be one of 64, 128, or 256")
    check_train_bf16({"key": key, "key_scale": key_scale, "learning_rate": learning_rate,
                      "learning_rate_scale": learning_rate_scale})
    if key.ndim != 3 or key.numel() == 0 or key.shape[-1] % head_size:
        raise ValueError("key must have non-empty shape [B,T,C], C divisible by head_size")
    if learning_rate.shape != key.shape:
        raise ValueError("learning_rate must match key")
    if key_scale.shape != (key.shape[-1],) or learning_rate_scale.shape != key_scale.shape:
        raise ValueError("kk-pre scale vectors must have shape [C]")


class _KKPre(torch.autograd.Function):
    @staticmethod
    def forward(ctx, key, key_scale, learning_rate, learning_rate_scale, head_size):
        outputs = extension().pretrain_tmix_kk_pre_forward(key, key_scale, learning_rate, learning_rate_scale,
                                                           head_size)
        ctx.save_for_backward(key, key_scale, learning_rate, learning_rate_scale, outputs[3])
        ctx.head_size = head_size
        return outputs[0], outputs[1], outputs[2]

    @staticmethod
    def backward(ctx, grad_new_key, grad_negative_direction, grad_scaled_direction):
        key, key_scale, learning_rate, learning_rate_scale, inverse_norm = ctx.saved_tensors
        zeros = None
        grads = []
        for g in (grad_new_key, grad_negative_direction, grad_scaled_direction):
            if g is None:
                zeros = torch.zeros_like(key) if zeros is None else zeros
                g = zeros
            grads.append(g.contiguous())
        gradients = extension().pretrain_tmix_kk_pre_backward(*grads, key, key_scale, learning_rate,
                                                              learning_rate_scale, inverse_norm, ctx.head_size)
        return tuple(g if needed else None for g, needed in zip(gradients, ctx.needs_input_grad[:4])) + (None,)


def pretrain_tmix_kk_pre_bf16(key, key_scale, learning_rate, learning_rate_scale, *, head_size=64):
    _check_inputs(key, key_scale, learning_rate, learning_rate_scale, head_size)
    return _KKPre.apply(key, key_scale, learning_rate, learning_rate_scale, head_size)


__all__ = ["pretrain_tmix_kk_pre_bf16"]
