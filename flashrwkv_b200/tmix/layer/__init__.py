"""A whole RWKV-7 TMix layer for a decode batch in one launch (no counterpart in the reference, whose layer is the
operator sequence mix6 -> projections -> kk_a_gate -> WKV7 -> lnx_rkvres_xg -> output projection).

`infer_tmix_decode_layer_forward_varlen` takes one token per sequence (1..8 rows, head size 64) and runs token shift,
the r / k / v and low-rank projections, the value-residual gate, kk_a_gate, the WKV7 step, the per-head
normalisation with bonus and gate, and the output projection as one persistent kernel whose stages are separated
by grid-wide barriers.  Intermediates are rounded to the io type where the separate operators round theirs, so the
result equals `reference_sequence` (the same layer through this package's separate operators) up to summation order.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..._ext import extension
from .._checks import check_io


@dataclass
class TMixLayerWeights:
    """Parameters of one TMix layer; every tensor 16-bit, contiguous, on the device of the activations.

    mix_r .. mix_g `[C]` (token-shift vectors); w_r, w_k, w_v, w_o `[C,C]` (original layout `[out,in]`);
    w1 / w2: rank-in `[R,C]` and rank-out `[C,R]` weights of the decay, a, gate and value-residual paths (dicts with
    keys "w", "a", "g", "v"); k_k, a0, k_a, r_k, ln_w, ln_b, v0 `[C]`.
    """
    mix_r: torch.Tensor
    mix_w: torch.Tensor
    mix_k: torch.Tensor
    mix_v: torch.Tensor
    mix_a: torch.Tensor
    mix_g: torch.Tensor
    w_r: torch.Tensor
    w_k: torch.Tensor
    w_v: torch.Tensor
    w_o: torch.Tensor
    w1: dict
    w2: dict
    k_k: torch.Tensor
    a0: torch.Tensor
    k_a: torch.Tensor
    r_k: torch.Tensor
    ln_w: torch.Tensor
    ln_b: torch.Tensor
    v0: torch.Tensor


_last_words: dict = {}


def decode_layer_error_flag():
    """The sticky device error flag of the last decode-layer launch (None before the first); non-zero after a
    grid-barrier wait ran out, in which case that launch's output is NaN.  Reading it synchronises."""
    words = _last_words.get("words")
    return None if words is None else int(words[7].item())


def infer_tmix_decode_layer_forward_varlen(x, v_first, weights: TMixLayerWeights, *, shift_state_pool, state_pool,
                                           cu_seqlens, state_indices, eps: float = 64e-5, validated_metadata=None):
    """`x`, `v_first` `[M,C]` (row m = the one new token of sequence m, 1 <= M <= 8) -> layer output `[M,C]`.

    `shift_state_pool [slots,C]` takes the rows of `x`; `state_pool [slots,C/64,64,64]` fp32 is advanced by one
    token in place.  `cu_seqlens` must be `arange(M+1)`; a ticket from `prepare_recurrent_metadata(..., max_seqlen=1)`
    skips the validation launch.
    """
    check_io("x", x, None)
    if x.ndim != 2 or not 1 <= x.shape[0] <= 8:
        raise ValueError("x must have packed shape [M,C] with 1 <= M <= 8 (one token per sequence)")
    check_io("v_first", v_first, x)
    if not isinstance(weights, TMixLayerWeights):
        raise TypeError("weights must be a TMixLayerWeights")
    if not isinstance(state_pool, torch.Tensor) or state_pool.dtype != torch.float32:
        raise TypeError("state_pool must be a float32 torch.Tensor")
    if not isinstance(eps, (int, float)) or not eps > 0:
        raise ValueError("eps must be positive")
    w = weights
    out, words = extension().tmix_decode_layer(
        x, v_first, shift_state_pool, state_pool, [w.mix_r, w.mix_w, w.mix_k, w.mix_v, w.mix_a, w.mix_g],
        [w.w_r, w.w_k, w.w_v, w.w_o], [w.w1[n] for n in "wagv"], [w.w2[n] for n in "wagv"],
        [w.k_k, w.a0, w.k_a, w.r_k, w.ln_w, w.ln_b, w.v0], cu_seqlens, state_indices, float(eps), validated_metadata)
    _last_words["words"] = words
    return out


def reference_sequence(x, v_first, weights: TMixLayerWeights, *, shift_state_pool, state_pool, cu_seqlens,
                       state_indices, eps: float = 64e-5, validated_metadata=None):
    """The same layer through the separate operators (the reference's operator sequence); any number of rows as long
    as every sequence has one token."""
    from .. import kk_a_gate, linear, lnx_rkvres_xg, mix6, wkv7

    w = weights
    M, C = x.shape
    xr, xw, xk, xv, xa, xg = mix6.infer_tmix_mix6_forward_varlen(
        x, w.mix_r, w.mix_w, w.mix_k, w.mix_v, w.mix_a, w.mix_g, shift_state_pool=shift_state_pool,
        cu_seqlens=cu_seqlens, state_indices=state_indices, max_seqlen=1, validated_metadata=validated_metadata)
    r_ = linear.infer_tmix_linear_forward_varlen(xr, w.w_r)
    k_ = linear.infer_tmix_linear_forward_varlen(xk, w.w_k)
    v_ = linear.infer_tmix_linear_forward_varlen(xv, w.w_v)
    fw, fa, fg, fv = linear.infer_tmix_lowrank_wagv_in_forward_varlen(xw, xa, xg, xv, w.w1["w"], w.w1["a"], w.w1["g"],
                                                                      w.w1["v"])
    w_, a12, g_, vres = linear.infer_tmix_lowrank_vres_forward_varlen(fw, fa, fg, fv, w.w2["w"], w.w2["a"], w.w2["g"],
                                                                      w.w2["v"], v_, v_first, w.v0)
    kk_, nkk, kka = kk_a_gate.infer_tmix_kk_a_gate_forward_varlen(k_, w.k_k, w.a0, a12, w.k_a)
    sh = (M, C // 64, 64)
    y = wkv7.infer_recurrent_fp32io16_forward_varlen(r_.view(sh), w_.view(sh), kk_.view(sh), vres.view(sh), nkk.view(sh),
                                                     kka.view(sh), state_pool=state_pool, cu_seqlens=cu_seqlens,
                                                     state_indices=state_indices, validated_metadata=validated_metadata,
                                                     max_seqlen=1)
    if eps != 64e-5:
        raise ValueError("the separate lnx_rkvres_xg operator has a fixed eps of 64e-5")
    z = lnx_rkvres_xg.infer_tmix_lnx_rkvres_xg_forward_varlen(y.view(M, C), r_, kk_, vres, w.r_k, w.ln_w, w.ln_b, g_)
    return linear.infer_tmix_linear_forward_varlen(z, w.w_o)


__all__ = ["TMixLayerWeights", "infer_tmix_decode_layer_forward_varlen", "reference_sequence",
           "decode_layer_error_flag"]
