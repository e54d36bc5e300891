"""Generate the golden vectors under tests/golden/ from the reference's own test oracles.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/FlashRWKV

The reference's oracles are pure PyTorch and run on CPU.  They are imported by
file path from the reference's ``tests/`` tree (nothing is copied); inputs are
seeded, rounded to the 16-bit io dtype where the case says so, and stored next
to the expected outputs so the tests do not depend on RNG stability.

Cases (reference file:line of the oracle that produced the expectation):
  recurrent_cfg0      tests/tmix/wkv7/test.py:157-213   B1 T64 H4 D64 fp32, S0 = 0
  recurrent_ragged    tests/tmix/wkv7/test.py:157-213   lengths (1,15,16,17,65), slots [5,0,7,2,4],
                      scales of tests/tmix/wkv7/test.py:417-477, bf16 io, with decay_bias
  recurrent_fp16state tests/tmix/wkv7/test.py:216-277   fp16 state pool with dither; lengths (1,2,4,8,19), slots
                      [5,0,7,2,4], elapsed = 11 * slot, value scales of tests/tmix/wkv7/test.py:417-477, fp16 io, bias
  recurrent_fp16state_d128  the same at head size 128: lengths (1,2,4), slots [3,0,2]
  chunk_bf16          tests/tmix/wkv7/chunk/test.py:18-49   lengths (1,9,17), scale 0.5, bf16 state
  rl_fp16             tests/rl_infctx/wkv7/test.py:12-53    lengths (2,5), fp16 io, decay_bias
  statetune           tests/tmix/wkv7/statetune/test.py:39-87 + autograd (:109-124), scale 0.75
  pretrain            tests/tmix/wkv7/pretrain/test.py:49-70 + autograd (:108-128), (B,T,H)=(2,32,2)
  tmix_*              formulas of tests/tmix/{mix6,kk_a_gate,lnx_rkvres_xg,vres_gate,linear,normalization}/test.py
"""
from __future__ import annotations

import argparse
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from flashrwkv_b200 import synthetic  # noqa: E402


def _load(reference: Path, rel: str, name: str):
    spec = importlib.util.spec_from_file_location(name, reference / rel)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def _save(name: str, **arrays) -> None:
    np.savez_compressed(HERE / f"{name}.npz", **{k: (_np(v) if isinstance(v, torch.Tensor) else np.asarray(v))
                                                 for k, v in arrays.items()})
    print("wrote", name, {k: tuple(np.asarray(_np(v) if isinstance(v, torch.Tensor) else v).shape)
                          for k, v in arrays.items()})


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the FlashRWKV reference checkout")
    ref = Path(ap.parse_args().reference)
    sys.path.insert(0, str(ref))
    wkv_test = _load(ref, "tests/tmix/wkv7/test.py", "ref_wkv7_test")
    chunk_test = _load(ref, "tests/tmix/wkv7/chunk/test.py", "ref_chunk_test")
    st_test = _load(ref, "tests/tmix/wkv7/statetune/test.py", "ref_statetune_test")
    pre_test = _load(ref, "tests/tmix/wkv7/pretrain/test.py", "ref_pretrain_test")
    rl_test = _load(ref, "tests/rl_infctx/wkv7/test.py", "ref_rl_test")

    # ---- recurrent_cfg0: benchmark configuration 0 through the reference oracle
    B, T, H, D = 1, 64, 4, 64
    toks = synthetic.wkv7_inputs(B * T, H, D, seed=20260804, dtype=torch.float32)
    cu, idx = synthetic.equal_length_metadata(B, T)
    pool = torch.zeros(B, H, D, D)
    y, final = wkv_test.rwkv7_decay_logits_reference(*toks, state_pool=pool, cu_seqlens=cu,
                                                     state_indices=idx)
    _save("recurrent_cfg0", r=toks[0], w=toks[1], k=toks[2], v=toks[3], a=toks[4], b=toks[5],
          cu_seqlens=cu, state_indices=idx, state_pool=pool, y=y, final_pool=final)

    # ---- recurrent_ragged: the reference's ragged case (value scales of its _make_case)
    torch.manual_seed(20260804 + 64 + 1)
    lengths = (1, 15, 16, 17, 65)
    N, H = sum(lengths), 2
    rnd = lambda s: (torch.randn(N, H, D) * s).to(torch.bfloat16)  # noqa: E731
    r, w, k, v, a, b = rnd(0.12), rnd(3.5), rnd(0.06), rnd(0.06), rnd(0.06), rnd(0.06)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
    idx = torch.tensor([5, 0, 7, 2, 4], dtype=torch.int32)
    pool = torch.randn(9, H, D, D) * 0.03
    bias = (torch.randn(H, D) * 0.2).to(torch.bfloat16)
    y, final = wkv_test.rwkv7_decay_logits_reference(r, w, k, v, a, b, state_pool=pool, cu_seqlens=cu,
                                                     state_indices=idx, scale=0.5, decay_bias=bias)
    _save("recurrent_ragged", r=r, w=w, k=k, v=v, a=a, b=b, cu_seqlens=cu, state_indices=idx,
          state_pool=pool, decay_bias=bias, scale=0.5, y=y, final_pool=final)

    # ---- recurrent_fp16state: the reference's fp16-state contract (dither, elapsed phase), its own value scales
    torch.manual_seed(20260804 + 64 + 7)
    lengths = (1, 2, 4, 8, 19)
    N, H = sum(lengths), 2
    rnd = lambda s: (torch.randn(N, H, D) * s).to(torch.float16)  # noqa: E731
    r, w, k, v, a, b = rnd(0.12), rnd(3.5), rnd(0.06), rnd(0.06), rnd(0.06), rnd(0.06)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
    idx = torch.tensor([5, 0, 7, 2, 4], dtype=torch.int32)
    pool = (torch.randn(9, H, D, D) * 0.03).half()
    elapsed = (torch.arange(9, dtype=torch.int32) * 11)
    bias = (torch.randn(H, D) * 0.2).to(torch.float16)
    y, final = wkv_test.rwkv7_fp16_reference(r, w, k, v, a, b, state_pool=pool, elapsed_state_pool=elapsed,
                                             cu_seqlens=cu, state_indices=idx, scale=0.5, decay_bias=bias)
    _save("recurrent_fp16state", r=r, w=w, k=k, v=v, a=a, b=b, cu_seqlens=cu, state_indices=idx, state_pool=pool,
          elapsed_state_pool=elapsed, decay_bias=bias, scale=0.5, y=y, final_pool=final)

    # ---- recurrent_fp16state_d128: the same contract at head size 128 (phase = head * 128 + channel + ...)
    torch.manual_seed(20260804 + 128 + 7)
    lengths = (1, 2, 4)
    N, H, D128 = sum(lengths), 2, 128
    rnd = lambda s: (torch.randn(N, H, D128) * s).to(torch.float16)  # noqa: E731
    r, w, k, v, a, b = rnd(0.12), rnd(3.5), rnd(0.06), rnd(0.06), rnd(0.06), rnd(0.06)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
    idx = torch.tensor([3, 0, 2], dtype=torch.int32)
    pool = (torch.randn(4, H, D128, D128) * 0.03).half()
    elapsed = (torch.arange(4, dtype=torch.int32) * 11)
    bias = (torch.randn(H, D128) * 0.2).to(torch.float16)
    y, final = wkv_test.rwkv7_fp16_reference(r, w, k, v, a, b, state_pool=pool, elapsed_state_pool=elapsed,
                                             cu_seqlens=cu, state_indices=idx, scale=0.5, decay_bias=bias)
    _save("recurrent_fp16state_d128", r=r, w=w, k=k, v=v, a=a, b=b, cu_seqlens=cu, state_indices=idx, state_pool=pool,
          elapsed_state_pool=elapsed, decay_bias=bias, scale=0.5, y=y, final_pool=final)

    # ---- chunk_bf16: ragged tail, bf16 state pool
    torch.manual_seed(11)
    lengths = [1, 9, 17]
    N = sum(lengths)
    ins = [(torch.randn(N, 1, D) * 0.02).to(torch.bfloat16) for _ in range(6)]
    cu = torch.tensor([0, 1, 10, 27], dtype=torch.int32)
    idx = torch.tensor([2, 0, 3], dtype=torch.int32)
    pool = (torch.randn(5, 1, D, D) * 0.002).to(torch.bfloat16)
    y, final = chunk_test._reference(*ins, pool, cu, idx, 0.5)
    _save("chunk_bf16", r=ins[0], w=ins[1], k=ins[2], v=ins[3], a=ins[4], b=ins[5], cu_seqlens=cu,
          state_indices=idx, state_pool=pool, scale=0.5, y=y, final_pool=final)

    # ---- rl_fp16: fp16 io, fp32 pool, decay bias
    torch.manual_seed(37)
    ins = [(torch.randn(7, 1, D) * 0.01).to(torch.float16) for _ in range(6)]
    pool = torch.randn(4, 1, D, D) * 0.01
    cu = torch.tensor([0, 2, 7], dtype=torch.int32)
    idx = torch.tensor([3, 1], dtype=torch.int32)
    bias = (torch.randn(1, D) * 0.01).to(torch.float16)
    y, final = rl_test._reference(*ins, state_pool=pool, cu_seqlens=cu, state_indices=idx, decay_bias=bias)
    _save("rl_fp16", r=ins[0], w=ins[1], k=ins[2], v=ins[3], a=ins[4], b=ins[5], cu_seqlens=cu,
          state_indices=idx, state_pool=pool, decay_bias=bias, y=y, final_pool=final)

    # ---- statetune: boundaries, state_dot_a and all seven gradients through autograd
    torch.manual_seed(20260805)
    Bs, Hs, Ns = 2, 1, 5
    S0 = (torch.randn(Bs, Hs, D, D) * 0.01).requires_grad_()
    vals = [(torch.randn(Ns, Hs, D).to(torch.float16) * 0.01).requires_grad_() for _ in range(6)]
    sco = torch.tensor([0, 2, 3], dtype=torch.int32)
    cs = torch.tensor([0, 1, 3], dtype=torch.int32)
    ce = torch.tensor([1, 3, 5], dtype=torch.int32)
    out, fin, bnd, sda = st_test._reference((S0, sco, cs, ce, *vals), 0.75)
    (out.float().square().sum() + fin.square().sum()).backward()
    _save("statetune", S0=S0, r=vals[0], w=vals[1], k=vals[2], v=vals[3], a=vals[4], b=vals[5],
          seq_chunk_offsets=sco, chunk_starts=cs, chunk_ends=ce, scale=0.75,
          y=out, final_state=fin, boundary=bnd, state_dot_a=sda,
          grad_output=(2.0 * out.float()).detach(), grad_final_state=(2.0 * fin).detach(),
          dS0=S0.grad, dr=vals[0].grad.float(), dw=vals[1].grad.float(), dk=vals[2].grad.float(),
          dv=vals[3].grad.float(), da=vals[4].grad.float(), db=vals[5].grad.float())

    # ---- pretrain: dense [B,T,C], zero S0, gradients through autograd
    Bp, Tp, Hp = 2, 32, 2
    torch.manual_seed(20260806 + Bp + Tp + Hp)
    vals = tuple((torch.randn(Bp, Tp, Hp * D).to(torch.bfloat16) * 0.05).requires_grad_() for _ in range(6))
    yp = pre_test._reference(vals)
    dy = torch.randn(Bp, Tp, Hp * D).to(torch.bfloat16)
    yp.backward(dy.float())
    _save("pretrain", r=vals[0], w=vals[1], k=vals[2], v=vals[3], a=vals[4], b=vals[5], y=yp, dy=dy,
          dr=vals[0].grad.float(), dw=vals[1].grad.float(), dk=vals[2].grad.float(),
          dv=vals[3].grad.float(), da=vals[4].grad.float(), db=vals[5].grad.float())

    # ---- TMix pieces: the expectations are the formulas the reference's tests evaluate inline
    # (tests/tmix/kk_a_gate/test.py:62-67, tests/tmix/lnx_rkvres_xg/test.py:50-63, tests/tmix/vres_gate/test.py:15-26,
    #  tests/tmix/mix6/test.py:263-278, tests/tmix/linear/test.py:395-424), evaluated here in fp32 on fp16 inputs
    torch.manual_seed(17)
    rows, heads, hs = 3, 2, 64
    C = heads * hs
    h16 = lambda *shape: torch.randn(*shape).to(torch.float16)  # noqa: E731
    k, k_k, a0, a12, k_a = h16(rows, C), h16(C), h16(C), h16(rows, C), h16(C)
    scaled = k.float().reshape(rows, heads, hs) * k_k.float().reshape(1, heads, hs)
    norm = scaled / scaled.square().sum(-1, keepdim=True).sqrt().clamp_min(1.0e-12)
    gate = torch.sigmoid(a0.float().reshape(1, heads, hs) + a12.float().reshape(rows, heads, hs))
    kaf = k_a.float().reshape(1, heads, hs)
    new_k = k.float().reshape(rows, heads, hs) * (gate * kaf + 1.0 - kaf)
    _save("tmix_kk_a_gate", k=k, k_k=k_k, a0=a0, a12=a12, k_a=k_a, new_k=new_k.reshape(rows, C),
          neg_kk=(-norm).reshape(rows, C), kka=(norm * gate).reshape(rows, C))

    torch.manual_seed(21)
    x, r, k, v, g = (h16(rows, C) for _ in range(5))
    r_k, weight, bias = h16(C), h16(C), h16(C)
    xf = x.float().reshape(rows, heads, hs)
    mean = xf.mean(-1, keepdim=True)
    rstd = (xf.var(-1, unbiased=False, keepdim=True) + 64.0e-5).rsqrt()
    resid = (r.float().reshape(rows, heads, hs) * k.float().reshape(rows, heads, hs)
             * r_k.float().reshape(1, heads, hs)).sum(-1, keepdim=True)
    out = ((xf - mean) * rstd * weight.float().reshape(1, heads, hs) + bias.float().reshape(1, heads, hs)
           + resid * v.float().reshape(rows, heads, hs)) * g.float().reshape(rows, heads, hs)
    _save("tmix_lnx", x=x, r=r, k=k, v=v, g=g, r_k=r_k, weight=weight, bias=bias, out=out.reshape(rows, C))

    torch.manual_seed(5)
    v, v_first, v12, v0 = h16(4, C), h16(4, C), h16(4, C), h16(C)
    out = v.float() + (v_first.float() - v.float()) * torch.sigmoid(v0.float() + v12.float())
    _save("tmix_vres", v=v, v_first=v_first, v12=v12, v0=v0, out=out)

    c = 8
    lengths = (2, 3)
    total = sum(lengths)
    x = torch.arange(total * c, dtype=torch.float16).reshape(total, c)
    params = [torch.full((c,), val, dtype=torch.float16) for val in (0.1, 0.2, 0.3, 0.4, 0.5, 0.6)]
    torch.manual_seed(3)
    initial = torch.randn(4, c).to(torch.float16)
    slots = [1, 3]
    expected = [[] for _ in range(6)]
    shift = initial.clone()
    start = 0
    for s, length in enumerate(lengths):
        previous = initial[slots[s]]
        for t in range(start, start + length):
            cur = x[t]
            for i, p in enumerate(params):
                expected[i].append((cur.float() + (previous.float() - cur.float()) * p.float()))
            previous = cur
        shift[slots[s]] = previous
        start += length
    _save("tmix_mix6", x=x, mix=torch.stack(params), shift_pool=initial,
          cu_seqlens=torch.tensor([0, 2, 5], dtype=torch.int32), state_indices=torch.tensor(slots, dtype=torch.int32),
          out=torch.stack([torch.stack(rows_) for rows_ in expected]), shift_after=shift)

    torch.manual_seed(9)
    M, Cc, R = 5, 256, 96
    xw, w1, w2 = h16(M, Cc), (torch.randn(R, Cc) * 0.05).to(torch.float16), (torch.randn(Cc, R) * 0.05).to(torch.float16)
    rank = (xw.float() @ w1.float().T).to(torch.float16)
    outw = torch.tanh(rank.float()) @ w2.float().T
    _save("tmix_lowrank", x=xw, w1=w1, w2=w2, rank=rank, out_tanh=outw)

    # ---- tmix_norm: add + LayerNorm family, formulas of tests/tmix/normalization/test.py:17-35 (F.layer_norm of the
    # rounded sum) and the fused add + LayerNorm + mix6 of tests/tmix/mix6/test.py:312-368 on three one-token rows
    torch.manual_seed(53)
    import torch.nn.functional as Fn
    rows, Cn = 3, 256
    xn = (torch.randn(rows, Cn) * 0.03).to(torch.float16)
    rn = (torch.randn(rows, Cn) * 0.02).to(torch.float16)
    wn = (torch.randn(Cn) * 0.1 + 1.0).to(torch.float16)
    bn = (torch.randn(Cn) * 0.01).to(torch.float16)
    params = [(torch.randn(Cn) * 0.1).to(torch.float16) for _ in range(6)]
    initial = torch.randn(5, Cn).to(torch.float16)
    slots = torch.tensor([3, 0, 4], dtype=torch.int32)
    summed = xn + rn                                               # fp16 add, as `x + residual` in the reference test
    ln_x = Fn.layer_norm(xn.float(), (Cn,), wn.float(), bn.float(), 1e-5)
    ln_sum = Fn.layer_norm(summed.float(), (Cn,), wn.float(), bn.float(), 1e-5)
    normalized = ln_sum.to(torch.float16)
    mixed = torch.stack([(normalized.float() + (initial[slots.long()].float() - normalized.float()) * p.float())
                         for p in params])
    shift_after = initial.clone()
    shift_after[slots.long()] = normalized
    _save("tmix_norm", x=xn, residual=rn, weight=wn, bias=bn, mix=torch.stack(params), shift_pool=initial,
          state_indices=slots, cu_seqlens=torch.arange(rows + 1, dtype=torch.int32), sum=summed, ln_x=ln_x,
          ln_sum=ln_sum, mixed=mixed, shift_after=shift_after)


if __name__ == "__main__":
    main()
