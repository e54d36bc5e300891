"""TEST INFRASTRUCTURE ONLY: float64 numpy restatement of the reference's training-side TMix glue, forward and backward.

Only tests/ may import this file; the product path never does.

Each function follows the arithmetic of one reference kernel pair (bf16 tensors widened to float, all sums in
float; here float64, so that the CUDA result can be judged against an exact value):

  a_gate         csrc/sm90/tmix/a_gate/pretrain_bf16_forward.cu, pretrain_bf16_backward.cu
  vres_gate      csrc/sm90/tmix/vres_gate/pretrain_bf16_forward.cu, pretrain_bf16_backward.cu
  mix6           csrc/sm90/tmix/mix6/pretrain_bf16_forward.cu, pretrain_bf16_backward.cu
                 (the torch formula of tests/tmix/mix6/test.py:72-77; StateTune form with an initial and a final
                 shift state: tests/tmix/mix6/test.py:114-118)
  kk_pre         csrc/sm90/tmix/kk_pre/pretrain_bf16_forward.cu:66-117 (eps 1e-12, clamp of the norm) and
                 pretrain_bf16_backward.cu (projection term only while the norm is above eps)
  lnx_rkvres_xg  csrc/sm90/tmix/lnx_rkvres_xg/pretrain_bf16_forward.cu:64-124 (eps 64e-5, biased variance; the
                 torch formula of tests/tmix/lnx_rkvres_xg/test.py:42-60)

Parity pin: the forwards are pinned to the formulas the reference's own tests evaluate (mix6, lnx, vres_gate, and
kk_a_gate = a_gate followed by kk_pre), stored as fixtures by tests/golden/make_golden.py and checked in
tests/test_tmix_train_oracle.py.  The reference's tests of the BACKWARDS hold no values (finiteness checks only), so
the backward functions here are pinned on the CPU against torch autograd (float64) of those formulas: for the
backward of a_gate, kk_pre and vres_gate that is all there is - parity unpinned by anything the reference holds.
"""
from __future__ import annotations

import numpy as np

NORMALIZE_EPS = 1.0e-12
LNX_EPS = 64e-5


def _f64(t) -> np.ndarray:
    if hasattr(t, "detach"):
        t = t.detach().double().cpu().numpy()
    return np.asarray(t, dtype=np.float64)


def _sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def _rows(t):
    return t.reshape(-1, t.shape[-1])


def a_gate(a0, a12):
    return _sigmoid(_f64(a0) + _f64(a12))


def a_gate_backward(grad_out, a0, a12):
    y = a_gate(a0, a12)
    d = _f64(grad_out) * y * (1.0 - y)
    return _rows(d).sum(0), d


def vres_gate(v, v_first, v0, v12):
    v, v_first = _f64(v), _f64(v_first)
    return v + (v_first - v) * _sigmoid(_f64(v0) + _f64(v12))


def vres_gate_backward(grad_out, v, v_first, v0, v12):
    g, v, v_first = _f64(grad_out), _f64(v), _f64(v_first)
    s = _sigmoid(_f64(v0) + _f64(v12))
    dz = g * (v_first - v) * s * (1.0 - s)
    return g * (1.0 - s), g * s, _rows(dz).sum(0), dz


def _shifted(x, initial=None):
    prev = np.zeros_like(x)
    prev[:, 1:] = x[:, :-1]
    if initial is not None:
        prev[:, 0] = _f64(initial)
    return prev


def mix6(x, mixes, initial=None):
    """`initial` = the StateTune form's shift state [B,C] (the row before t = 0); None = zero (pretrain form)."""
    x = _f64(x)
    xx = _shifted(x, initial) - x
    return [x + xx * _f64(m) for m in mixes]


def mix6_backward(grad_outs, x, mixes, initial=None, grad_final=None):
    """Returns (grad_x, [grad_mix] * 6, grad_initial); grad_final = the gradient of the final shift state x[:, -1]."""
    x = _f64(x)
    xx = _shifted(x, initial) - x
    gx = np.zeros_like(x)
    ginit = np.zeros_like(x[:, 0])
    gm = []
    for g, m in zip(grad_outs, mixes):
        g, m = _f64(g), _f64(m)
        gx += g * (1.0 - m)
        gx[:, :-1] += (g * m)[:, 1:]
        ginit += (g * m)[:, 0]
        gm.append(_rows(g * xx).sum(0))
    if grad_final is not None:
        gx[:, -1] += _f64(grad_final)
    return gx, gm, ginit


def _heads(t, head_size):
    return t.reshape(*t.shape[:-1], t.shape[-1] // head_size, head_size)


def kk_pre(k, k_k, a, k_a, head_size=64):
    k, k_k, a, k_a = _f64(k), _f64(k_k), _f64(a), _f64(k_a)
    u = _heads(k * k_k, head_size)
    inv = 1.0 / np.maximum(np.sqrt((u * u).sum(-1, keepdims=True)), NORMALIZE_EPS)
    kk = (u * inv).reshape(k.shape)
    return k * (1.0 + (a - 1.0) * k_a), -kk, kk * a, inv[..., 0]


def kk_pre_backward(g_new_k, g_neg_kk, g_kka, k, k_k, a, k_a, head_size=64):
    g_new_k, g_neg_kk, g_kka = _f64(g_new_k), _f64(g_neg_kk), _f64(g_kka)
    k, k_k, a, k_a = _f64(k), _f64(k_k), _f64(a), _f64(k_a)
    _, neg_kk, _, inv = kk_pre(k, k_k, a, k_a, head_size)
    kk = -neg_kk
    gkk = -g_neg_kk + g_kka * a
    dot = (_heads(kk, head_size) * _heads(gkk, head_size)).sum(-1, keepdims=True)
    dot = np.where(inv[..., None] < 1.0 / NORMALIZE_EPS, dot, 0.0)
    gu = (inv[..., None] * (_heads(gkk, head_size) - _heads(kk, head_size) * dot)).reshape(k.shape)
    gk = g_new_k * (1.0 + (a - 1.0) * k_a) + gu * k_k
    ga = g_new_k * k * k_a + g_kka * kk
    return gk, _rows(gu * k).sum(0), ga, _rows(g_new_k * k * (a - 1.0)).sum(0)


def lnx_rkvres_xg(x, r, k, v, r_k, weight, bias, g, head_size=64):
    x, r, k, v, g = (_f64(t) for t in (x, r, k, v, g))
    r_k, weight, bias = (_f64(t).reshape(-1) for t in (r_k, weight, bias))
    xh = _heads(x, head_size)
    mean = xh.mean(-1, keepdims=True)
    rstd = 1.0 / np.sqrt(((xh - mean) ** 2).mean(-1, keepdims=True) + LNX_EPS)
    xhat = ((xh - mean) * rstd).reshape(x.shape)
    s = _heads(r * k * r_k, head_size).sum(-1, keepdims=True)
    pre = xhat * weight + bias + (s * _heads(v, head_size)).reshape(x.shape)
    return pre * g, mean[..., 0], rstd[..., 0]


def lnx_rkvres_xg_backward(grad_out, x, r, k, v, r_k, weight, bias, g, head_size=64):
    go, x, r, k, v, g = (_f64(t) for t in (grad_out, x, r, k, v, g))
    shape_rk = np.asarray(_f64(r_k)).shape
    r_k, weight, bias = (_f64(t).reshape(-1) for t in (r_k, weight, bias))
    xh = _heads(x, head_size)
    mean = xh.mean(-1, keepdims=True)
    rstd = 1.0 / np.sqrt(((xh - mean) ** 2).mean(-1, keepdims=True) + LNX_EPS)
    xhat = (xh - mean) * rstd
    s = _heads(r * k * r_k, head_size).sum(-1, keepdims=True)
    pre = xhat.reshape(x.shape) * weight + bias + (s * _heads(v, head_size)).reshape(x.shape)
    gg = go * pre
    gy = go * g
    gw = _rows(gy * xhat.reshape(x.shape)).sum(0)
    gb = _rows(gy).sum(0)
    gv = (_heads(gy, head_size) * s).reshape(x.shape)
    gs = (_heads(gy, head_size) * _heads(v, head_size)).sum(-1, keepdims=True)
    gr = (gs * _heads(k * r_k, head_size)).reshape(x.shape)
    gk = (gs * _heads(r * r_k, head_size)).reshape(x.shape)
    grk = _rows((gs * _heads(r * k, head_size)).reshape(x.shape)).sum(0).reshape(shape_rk)
    gxh = _heads(gy * weight, head_size)
    gx = rstd * (gxh - gxh.mean(-1, keepdims=True) - xhat * (gxh * xhat).mean(-1, keepdims=True))
    return gx.reshape(x.shape), gr, gk, gv, grk, gw, gb, gg
