"""TMix projections: dense C x C linears and the low-rank (rank-in / rank-out) group.

Mirror of the reference's `flashrwkv2/tmix/linear/__init__.py:25-482` (names, positional/keyword split, the
`R <= 512` limit).  Every operator here is `act(x) @ W^T` with `W` in the reference's *original* layout `[N,K]`;
groups of three or four projections go to the device in one launch.  A weight given only in the reference's
*runtime* layout `[K,N]` (`weight_is_transposed=True`, the `*_runtime` arguments) is read in place by kernels of
its own (a small-row kernel, and the TMA GEMM with an MN-major operand): no transposed copy is made.
fp16 as in the reference, bf16 in addition.
"""
from __future__ import annotations

import torch

from ..._ext import extension
from .._checks import check_io

_ACT = {"none": 0, "tanh": 1, "sigmoid": 2}
LOWRANK_LIMIT = 512


def _check_x(x, name="x", ref=None):
    check_io(name, x, ref)
    if x.ndim != 2 or x.shape[0] <= 0 or x.shape[1] <= 0:
        raise ValueError(f"{name} must have packed shape [M,K]")


def _original(name, original, runtime, x, *, rank_dim: int | None, input_projection: bool):
    """Validate the weight(s) of `x @ W^T`; returns `(original [N,K] or None, runtime [K,N] or None)`."""
    if original is None and runtime is None:
        raise ValueError(f"{name}: an original-layout or a runtime-layout weight is required")
    if original is not None:
        check_io(name, original, x)
        if original.ndim != 2 or original.shape[1] != x.shape[1]:
            raise ValueError(f"{name} must have original layout [N,K] with K = {x.shape[1]}")
    if runtime is not None:
        check_io(f"{name}_runtime", runtime, x)
        if runtime.ndim != 2 or runtime.shape[0] != x.shape[1]:
            raise ValueError(f"{name}_runtime must have runtime layout [K,N] with K = {x.shape[1]}")
        if original is not None and runtime.shape != (original.shape[1], original.shape[0]):
            raise ValueError(f"{name}_runtime must be the [K,N] transpose of {name}")
    if rank_dim is not None:
        if original is not None:
            rank = original.shape[0] if input_projection else original.shape[1]
        else:
            rank = runtime.shape[1] if input_projection else runtime.shape[0]
        if rank > rank_dim:
            raise ValueError(f"{name}: low-rank dimension {rank} exceeds R <= {rank_dim}")
    return original, runtime


def _grouped(xs, weights, acts, vres=None):
    """`weights`: one `(original, runtime)` pair (or a plain original-layout tensor) per projection.  All-original groups leave in one launch; a
    projection that has only the runtime layout takes the kernels that read `[K,N]` in place."""
    C = extension()
    codes = [_ACT[a] for a in acts]
    weights = [w if isinstance(w, tuple) else (w, None) for w in weights]
    if all(o is not None for o, _ in weights):
        return C.tmix_linear_grouped(list(xs), [o for o, _ in weights], codes, vres)
    outs = []
    for i, (x, (o, r)) in enumerate(zip(xs, weights)):
        one = vres if i + 1 == len(xs) else None
        if o is not None:
            outs.append(C.tmix_linear_grouped([x], [o], [codes[i]], one)[0])
        else:
            outs.append(C.tmix_linear_runtime_layout(x, r, codes[i], one))
    return outs


# ---- dense linears ----------------------------------------------------------------------------------------
def infer_tmix_linear_forward_varlen(x, weight, *, weight_is_transposed: bool = False):
    """`x [M,K] @ weight[N,K]^T -> [M,N]`; with `weight_is_transposed` the weight is `[K,N]` and `x @ weight`."""
    _check_x(x)
    if weight_is_transposed:
        w = _original("weight", None, weight, x, rank_dim=None, input_projection=True)
    else:
        w = _original("weight", weight, None, x, rank_dim=None, input_projection=True)
    return _grouped([x], [w], ["none"])[0]


def infer_tmix_linear_attention_c2c_forward_varlen(x, weight):
    return infer_tmix_linear_forward_varlen(x, weight)


def infer_tmix_linear_ffn_key_forward_varlen(x, weight):
    return infer_tmix_linear_forward_varlen(x, weight)


def _linear_t(x, weight_t, act):
    _check_x(x)
    if x.shape[0] > 65535:
        raise ValueError("M must be at most 65535")
    w = _original("weight_t", weight_t, None, x, rank_dim=None, input_projection=True)
    return _grouped([x], [w], [act])[0]


def infer_tmix_linear_t_forward_varlen(x, weight_t):
    return _linear_t(x, weight_t, "none")


def infer_tmix_linear_t_tanh_forward_varlen(x, weight_t):
    return _linear_t(x, weight_t, "tanh")


def infer_tmix_linear_t_sigmoid_forward_varlen(x, weight_t):
    return _linear_t(x, weight_t, "sigmoid")


def infer_tmix_linear_t_vres_forward_varlen(x, weight_t, v, v_first, v0):
    _check_x(x)
    w = _original("weight_t", weight_t, None, x, rank_dim=None, input_projection=True)
    return _grouped([x], [w], ["none"], (v, v_first, v0))[0]


def _act(x, code):
    _check_x(x)
    if x.numel() % 2:
        raise ValueError("x must have an even element count")
    if x.numel() % 8:
        raise ValueError("this build needs an element count that is a multiple of 8")
    return extension().tmix_act_forward(x, code)


def infer_tmix_linear_act_tanh_forward_varlen(x):
    return _act(x, 1)


def infer_tmix_linear_act_sigmoid_forward_varlen(x):
    return _act(x, 2)


# ---- single low-rank projections ----------------------------------------------------------------------------
def _rank(x, weight, weight_t, act, input_projection):
    _check_x(x)
    w = _original("weight_t", weight_t, weight, x, rank_dim=LOWRANK_LIMIT, input_projection=input_projection)
    return _grouped([x], [w], [act])[0]


def infer_tmix_linear_rank_in_forward_varlen(x, weight=None, weight_t=None):
    return _rank(x, weight, weight_t, "none", True)


def infer_tmix_linear_rank_out_forward_varlen(x, weight=None, weight_t=None):
    return _rank(x, weight, weight_t, "none", False)


def infer_tmix_linear_rank_out_tanh_forward_varlen(x, weight=None, weight_t=None):
    return _rank(x, weight, weight_t, "tanh", False)


def infer_tmix_linear_rank_out_sigmoid_forward_varlen(x, weight=None, weight_t=None):
    return _rank(x, weight, weight_t, "sigmoid", False)


# ---- the composite low-rank group ----------------------------------------------------------------------------
def _rows(named):
    first = named[0][1]
    for name, t in named:
        _check_x(t, name, None if t is first else first)
        if t.shape[0] != first.shape[0]:
            raise ValueError(f"{name} must have {first.shape[0]} packed rows")


def infer_tmix_lowrank_in_forward_varlen(x_w, x_a, x_g, w1, a1, g1, *, w1_runtime=None, a1_runtime=None,
                                         g1_runtime=None):
    """Rank-in for decay / a / gate: three `[M,C] @ [R,C]^T -> [M,R]` in one launch."""
    _rows([("x_w", x_w), ("x_a", x_a), ("x_g", x_g)])
    ws = [_original(n, o, r, x, rank_dim=LOWRANK_LIMIT, input_projection=True)
          for n, o, r, x in (("w1", w1, w1_runtime, x_w), ("a1", a1, a1_runtime, x_a), ("g1", g1, g1_runtime, x_g))]
    return tuple(_grouped([x_w, x_a, x_g], ws, ["none"] * 3))


def infer_tmix_lowrank_wagv_in_forward_varlen(x_w, x_a, x_g, x_v, w1, a1, g1, v1, *, w1_runtime=None,
                                              a1_runtime=None, g1_runtime=None, v1_runtime=None):
    """Rank-in for decay / a / gate / value-residual in one launch."""
    _rows([("x_w", x_w), ("x_a", x_a), ("x_g", x_g), ("x_v", x_v)])
    ws = [_original(n, o, r, x, rank_dim=LOWRANK_LIMIT, input_projection=True)
          for n, o, r, x in (("w1", w1, w1_runtime, x_w), ("a1", a1, a1_runtime, x_a), ("g1", g1, g1_runtime, x_g),
                             ("v1", v1, v1_runtime, x_v))]
    return tuple(_grouped([x_w, x_a, x_g, x_v], ws, ["none"] * 4))


def infer_tmix_lowrank_out_forward_varlen(w1, a1, g1, w2, a2, g2, *, w2_runtime=None, a2_runtime=None,
                                          g2_runtime=None):
    """Rank-out: `tanh(w1) @ w2^T`, `a1 @ a2^T`, `sigmoid(g1) @ g2^T` (weights `[C,R]`) in one launch."""
    _rows([("w1", w1), ("a1", a1), ("g1", g1)])
    ws = [_original(n, o, r, x, rank_dim=LOWRANK_LIMIT, input_projection=False)
          for n, o, r, x in (("w2", w2, w2_runtime, w1), ("a2", a2, a2_runtime, a1), ("g2", g2, g2_runtime, g1))]
    return tuple(_grouped([w1, a1, g1], ws, ["tanh", "none", "sigmoid"]))


def infer_tmix_lowrank_vres_forward_varlen(w1, a1, g1, v1, w2, a2, g2, v2, v, v_first, v0, *, w2_runtime=None,
                                           a2_runtime=None, g2_runtime=None, v2_runtime=None):
    """Rank-out for W/A/G plus the value path with its residual gate fused: `v + (v_first - v) * sigmoid(v0 + v1 @ v2^T)`."""
    _rows([("w1", w1), ("a1", a1), ("g1", g1), ("v1", v1)])
    ws = [_original(n, o, r, x, rank_dim=LOWRANK_LIMIT, input_projection=False)
          for n, o, r, x in (("w2", w2, w2_runtime, w1), ("a2", a2, a2_runtime, a1), ("g2", g2, g2_runtime, g1),
                             ("v2", v2, v2_runtime, v1))]
    for name, t in (("v", v), ("v_first", v_first), ("v0", v0)):
        check_io(name, t, w1)
    return tuple(_grouped([w1, a1, g1, v1], ws, ["tanh", "none", "sigmoid", "none"], (v, v_first, v0)))


__all__ = [n for n in dir() if n.startswith("infer_tmix_")]
