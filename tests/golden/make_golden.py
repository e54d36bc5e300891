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
  chunk_bf16          tests/tmix/wkv7/chunk/test.py:18-49   lengths (1,9,17), scale 0.5, bf16 state
  rl_fp16             tests/rl_infctx/wkv7/test.py:12-53    lengths (2,5), fp16 io, decay_bias
  statetune           tests/tmix/wkv7/statetune/test.py:39-87 + autograd (:109-124), scale 0.75
  pretrain            tests/tmix/wkv7/pretrain/test.py:49-70 + autograd (:108-128), (B,T,H)=(2,32,2)
  tmix_*              formulas of tests/tmix/{mix6,kk_a_gate,lnx_rkvres_xg,vres_gate,linear}/test.py
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
    ap.add_argument("--reference", default="/root/reference")
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


if __name__ == "__main__":
    main()
