"""CPU oracle for the WKV7 time-mix path.  TEST INFRASTRUCTURE ONLY.

Two restatements of the reference's arithmetic live here:

* ``forward_torch`` -- a pure-PyTorch fp32 recurrence with the same structure as
  the reference's test oracle (``tests/tmix/wkv7/test.py:157-213`` in the
  reference project): a Python loop over sequences and tokens, vectorised over
  heads.  It is what the benchmark times as the CPU baseline.
* the C functions of ``wkv7_oracle.c`` (loaded through ctypes), used by the
  parity tests because they finish large cases in seconds.

Nothing in the product package imports this module.  Parity is pinned by
``tests/test_oracle_golden.py`` against vectors generated from the reference's
own oracles (``tests/golden/make_golden.py``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle_wkv7.so"
_lib = None

DECAY_RATE = 0.6065306597126334  # exp(-0.5)


def build(force: bool = False) -> Path:
    """Compile the C oracle next to its source (gcc, OpenMP)."""
    import hashlib

    src = _HERE / "wkv7_oracle.c"
    digest = hashlib.sha256(src.read_bytes() + (_HERE / "Makefile").read_bytes()).hexdigest()
    stamp = _HERE / "liboracle_wkv7.so.stamp"
    if force or not _LIB_PATH.exists() or not stamp.exists() or stamp.read_text().strip() != digest:
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle_wkv7.so"], check=True,
                       stdout=subprocess.DEVNULL)
        stamp.write_text(digest + "\n")
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(_load().oracle_num_threads())


def set_num_threads(n: int) -> None:
    _load().oracle_set_num_threads(int(n))


def _f32(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        x = x.detach().float().cpu().numpy()
    return np.ascontiguousarray(x, dtype=np.float32)


def _i32(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().numpy()
    return np.ascontiguousarray(x, dtype=np.int32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def retention(logits) -> np.ndarray:
    """w = exp(-exp(-0.5) * sigmoid(x)) (csrc/sm120/tmix/wkv7/recurrent_decay.cuh:18-22)."""
    x = _f32(logits)
    out = np.empty_like(x)
    _load().oracle_retention_f32(_p(x), _p(out), ctypes.c_int64(x.size))
    return out


def forward(r, decay_logits, k, v, a, b, *, state_pool, cu_seqlens, state_indices=None,
            scale: float = 1.0, decay_bias=None, chunks=None, want_state_dot_a: bool = False,
            double: bool = True, inplace: bool = False):
    """Packed varlen WKV7 forward.

    Returns a dict with ``y`` [N,H,D], ``state_pool`` (updated copy), and, when
    ``chunks=(seq_chunk_offsets, chunk_starts, chunk_ends)`` is given,
    ``boundary`` [Cn,H,D,D] (state before each chunk); ``state_dot_a`` [N,H,D]
    when requested.  ``double`` selects float64 accumulation.  ``inplace`` updates a
    contiguous float32 ndarray ``state_pool`` directly instead of a copy.
    """
    lib = _load()
    r, w, k, v, a, b = (_f32(t) for t in (r, decay_logits, k, v, a, b))
    N, H, D = r.shape
    if D > 256:
        raise ValueError("oracle supports D <= 256")
    if inplace:
        pool = state_pool
        if not (isinstance(pool, np.ndarray) and pool.dtype == np.float32 and pool.flags.c_contiguous):
            raise TypeError("inplace needs a C-contiguous float32 ndarray state_pool")
    else:
        pool = _f32(state_pool).copy()
    cu = _i32(cu_seqlens)
    B = cu.size - 1
    idx = None if state_indices is None else _i32(state_indices)
    bias = None if decay_bias is None else _f32(decay_bias).reshape(H, D)
    y = np.empty_like(r)
    sco = cs = ce = bnd = None
    if chunks is not None:
        sco, cs, ce = (_i32(t) for t in chunks)
        bnd = np.zeros((cs.size, H, D, D), dtype=np.float32)
    sda = np.zeros_like(r) if want_state_dot_a else None
    fn = lib.oracle_wkv7_forward_f64 if double else lib.oracle_wkv7_forward_f32
    fn(_p(cu), _p(idx), _p(sco), _p(cs), _p(ce), ctypes.c_int(B), ctypes.c_int(H),
       ctypes.c_int(D), _p(pool), _p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(bias),
       ctypes.c_float(scale), _p(y), _p(bnd), _p(sda))
    return {"y": y, "state_pool": pool, "boundary": bnd, "state_dot_a": sda}


def forward_fp16(r, decay_logits, k, v, a, b, *, state_pool, elapsed_state_pool, cu_seqlens, state_indices=None,
                 scale: float = 1.0, decay_bias=None):
    """Packed varlen WKV7 forward on an fp16 state pool (rounded retention increment with dither).

    ``state_pool`` is a float16 tensor / array ``[slots,H,D,D]``.  Returns ``y`` (float32 array holding the
    fp16-rounded outputs) and ``state_pool`` (updated float16 copy).  ``elapsed_state_pool`` int32 ``[slots]``.
    """
    lib = _load()
    r, w, k, v, a, b = (_f32(t) for t in (r, decay_logits, k, v, a, b))
    N, H, D = r.shape
    if D > 256:
        raise ValueError("oracle supports D <= 256")
    if hasattr(state_pool, "detach"):
        state_pool = state_pool.detach().cpu().numpy()
    pool = np.ascontiguousarray(state_pool, dtype=np.float16).copy()
    cu = _i32(cu_seqlens)
    idx = None if state_indices is None else _i32(state_indices)
    elapsed = _i32(elapsed_state_pool)
    bias = None if decay_bias is None else _f32(decay_bias).reshape(H, D)
    y = np.empty_like(r)
    lib.oracle_wkv7_fp16_forward(_p(cu), _p(idx), _p(elapsed), ctypes.c_int(cu.size - 1), ctypes.c_int(H),
                                 ctypes.c_int(D), _p(pool), _p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(bias),
                                 ctypes.c_float(scale), _p(y))
    return {"y": y, "state_pool": pool}


def backward(r, decay_logits, k, v, a, b, *, initial_state, cu_seqlens, grad_output,
             grad_final_state=None, scale: float = 1.0, decay_bias=None):
    """Gradients of ``forward`` (float64 accumulation); initial_state is [B,H,D,D]."""
    lib = _load()
    r, w, k, v, a, b = (_f32(t) for t in (r, decay_logits, k, v, a, b))
    N, H, D = r.shape
    S0 = _f32(initial_state)
    cu = _i32(cu_seqlens)
    B = cu.size - 1
    dy = _f32(grad_output)
    dSf = None if grad_final_state is None else _f32(grad_final_state)
    bias = None if decay_bias is None else _f32(decay_bias).reshape(H, D)
    outs = [np.zeros_like(r) for _ in range(6)]
    dS0 = np.zeros_like(S0)
    lib.oracle_wkv7_backward_f64(_p(cu), ctypes.c_int(B), ctypes.c_int(H), ctypes.c_int(D),
                                 _p(S0), _p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(bias),
                                 ctypes.c_float(scale), _p(dy), _p(dSf),
                                 *(_p(o) for o in outs), _p(dS0))
    names = ("r", "decay_logits", "k", "v", "a", "b")
    grads = dict(zip(names, outs))
    grads["initial_state"] = dS0
    return grads


def forward_torch(r, decay_logits, k, v, a, b, *, state_pool, cu_seqlens, state_indices,
                  scale: float = 1.0, decay_bias=None):
    """Pure-PyTorch fp32 recurrence, token by token, vectorised over heads."""
    N, H, D = r.shape
    pool = state_pool.float().clone()
    cu = [int(x) for x in cu_seqlens.tolist()]
    slots = [int(x) for x in state_indices.tolist()]
    rf, wf, kf, vf, af, bf = (t.float() for t in (r, decay_logits, k, v, a, b))
    if decay_bias is not None:
        wf = wf + decay_bias.float().reshape(1, H, D)
    ret = torch.exp(-DECAY_RATE * torch.sigmoid(wf))
    y = torch.empty((N, H, D), dtype=torch.float32)
    for s, slot in enumerate(slots):
        S = pool[slot].clone()
        for t in range(cu[s], cu[s + 1]):
            sa = torch.einsum("hk,hkv->hv", af[t], S)
            S = ret[t].unsqueeze(-1) * S + bf[t].unsqueeze(-1) * sa.unsqueeze(-2) \
                + kf[t].unsqueeze(-1) * vf[t].unsqueeze(-2)
            y[t] = scale * torch.einsum("hk,hkv->hv", rf[t], S)
        pool[slot] = S
    return y, pool


# --------------------------------------------------------------------------- TMix pieces

def mix6(x, shift_pool, mixes, cu_seqlens, state_indices):
    x = _f32(x)
    N, C = x.shape
    pool = _f32(shift_pool).copy()
    mix = np.stack([_f32(m) for m in mixes])
    cu, idx = _i32(cu_seqlens), _i32(state_indices)
    out = np.empty((6, N, C), dtype=np.float32)
    _load().oracle_mix6(_p(x), _p(pool), _p(mix), _p(cu), _p(idx), ctypes.c_int(idx.size),
                        ctypes.c_int(C), _p(out), ctypes.c_int64(N))
    return out, pool


def kk_a_gate(k, k_k, a0, a12, k_a, head_size: int = 64):
    k, k_k, a0, a12, k_a = (_f32(t) for t in (k, k_k, a0, a12, k_a))
    N, C = k.shape
    outs = [np.empty_like(k) for _ in range(3)]
    _load().oracle_kk_a_gate(_p(k), _p(k_k), _p(a0), _p(a12), _p(k_a), ctypes.c_int64(N),
                             ctypes.c_int(C // head_size), ctypes.c_int(head_size),
                             *(_p(o) for o in outs))
    return tuple(outs)


def lnx_rkvres_xg(x, r, k, v, r_k, weight, bias, g, head_size: int = 64, eps: float = 64e-5):
    x, r, k, v, r_k, weight, bias, g = (_f32(t) for t in (x, r, k, v, r_k, weight, bias, g))
    N, C = x.shape
    out = np.empty_like(x)
    _load().oracle_lnx_rkvres_xg(_p(x), _p(r), _p(k), _p(v), _p(r_k), _p(weight), _p(bias),
                                 _p(g), ctypes.c_int64(N), ctypes.c_int(C // head_size),
                                 ctypes.c_int(head_size), ctypes.c_double(eps), _p(out))
    return out


def vres_gate(v, v_first, v0, v12):
    v, v_first, v0, v12 = (_f32(t) for t in (v, v_first, v0, v12))
    N, C = v.shape
    out = np.empty_like(v)
    _load().oracle_vres_gate(_p(v), _p(v_first), _p(v0), _p(v12), ctypes.c_int64(N),
                             ctypes.c_int(C), _p(out))
    return out


def linear_nt(x, weight, act: str = "none"):
    """y = act(x) @ weight.T with weight [N,K]; act in {none,tanh,sigmoid}."""
    x, weight = _f32(x), _f32(weight)
    M, K = x.shape
    Nn = weight.shape[0]
    y = np.empty((M, Nn), dtype=np.float32)
    code = {"none": 0, "tanh": 1, "sigmoid": 2}[act]
    _load().oracle_linear_nt(_p(x), _p(weight), ctypes.c_int64(M), ctypes.c_int(Nn),
                             ctypes.c_int(K), ctypes.c_int(code), _p(y))
    return y


def layer_norm(x, weight, bias, eps: float = 1e-5, residual=None, io_dtype=None):
    """`LayerNorm(x [+ residual])` over the last axis in float64 (biased variance), the formula of the reference's
    normalization tests (tests/tmix/normalization/test.py:17-35: `F.layer_norm` of the summed rows).  With `residual`
    returns `(sum, normalized)`; `io_dtype` rounds the sum first, as the kernels' returned sum tensor is."""
    xs = _f32(x).astype(np.float64)
    if residual is not None:
        xs = xs + _f32(residual).astype(np.float64)
        if io_dtype is not None:
            xs = torch.from_numpy(xs).to(io_dtype).double().numpy()
    mean = xs.mean(axis=-1, keepdims=True)
    var = ((xs - mean) ** 2).mean(axis=-1, keepdims=True)
    out = (xs - mean) / np.sqrt(var + eps) * _f32(weight).astype(np.float64) + _f32(bias).astype(np.float64)
    out = out.astype(np.float32)
    return (xs.astype(np.float32), out) if residual is not None else out

