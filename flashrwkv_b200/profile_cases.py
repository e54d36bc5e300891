"""Small, self-contained workloads for profiler captures: `python -m flashrwkv_b200.profile_cases <case>`.

Each case holds well under a few GB on the device, uses inputs larger than the 126 MB L2 where DRAM figures
matter, runs a handful of launches and exits, so that an `ncu` capture of one of its kernels ends by itself.

  chunk   chunked forward (build + scan): B=2, T=4096, H=32  (4096 (chunk, head) items)
  train   StateTune forward + backward: B=2, T=2048, H=32
  train512  the same at B=8, T=512, H=64: 512 (sequence, head) pairs, the occupancy of the benchmark's training shape
  tmix    one TMix layer chain at C=2048 for M in (4, 512)
  decode  recurrent decode steps at B=256, H=32 (the benchmark's shape, 8 launches)
  decode16  the same on an fp16 state pool
  glue    training-side TMix glue, forward + backward of the five operators: B=2, T=4096, C=4096 (67 MB per tensor)
"""
from __future__ import annotations

import sys

import torch

import flashrwkv_b200 as F
from flashrwkv_b200 import synthetic
from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

D = 64


def case_chunk(reps: int = 3):
    B, T, H = 2, 4096, 32
    toks = [t.cuda() for t in synthetic.wkv7_inputs(B * T, H, D, seed=1)]
    cu, _ = synthetic.equal_length_metadata(B, T, device="cuda")
    pool = synthetic.state_pool(B, H, D, seed=2, device="cuda")
    meta = make_chunk_metadata(cu, 64)
    for _ in range(reps):
        wkv7_chunk_forward(*toks, state=pool, chunk_metadata=meta)


def case_train(reps: int = 2, B: int = 2, T: int = 2048, H: int = 32):
    toks = [t.cuda().requires_grad_() for t in synthetic.wkv7_inputs(B * T, H, D, seed=3)]
    S0 = synthetic.state_pool(B, H, D, seed=4, device="cuda").requires_grad_()
    cu, _ = synthetic.equal_length_metadata(B, T, device="cuda")
    meta = make_chunk_metadata(cu, 64)
    dy = torch.randn(B * T, H, D, device="cuda").to(torch.bfloat16)
    for _ in range(reps):
        out = F.statetune_recurrent_fp32io16(S0, *meta, *toks)
        out[0].backward(dy)


def case_tmix(reps: int = 3):
    C, H = 2048, 32
    g = torch.Generator().manual_seed(3)
    wt = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).cuda()  # noqa: E731
    ranks = {"w": 96, "a": 96, "g": 256, "v": 64}
    Wr = wt(C, C)
    w1 = {n: wt(r, C) for n, r in ranks.items()}
    w2 = {n: wt(C, r) for n, r in ranks.items()}
    v0 = torch.rand(C, generator=g).to(torch.bfloat16).cuda()
    for M in (4, 512):
        xs = [torch.randn(M, C, generator=g).to(torch.bfloat16).cuda() for _ in range(6)]
        for _ in range(reps):
            F.infer_tmix_linear_forward_varlen(xs[0], Wr)
            feats = F.infer_tmix_lowrank_wagv_in_forward_varlen(xs[1], xs[2], xs[3], xs[4], w1["w"], w1["a"], w1["g"],
                                                                w1["v"])
            F.infer_tmix_lowrank_vres_forward_varlen(*feats, w2["w"], w2["a"], w2["g"], w2["v"], xs[4], xs[5], v0)


def case_decode(reps: int = 8):
    B, H = 256, 32
    cu, idx = synthetic.equal_length_metadata(B, 1, device="cuda")
    pool = synthetic.state_pool(B, H, D, seed=5, device="cuda")
    toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=6)]
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B, max_seqlen=1)
    for _ in range(reps):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                  validated_metadata=ticket, max_seqlen=1)


def case_decode16(reps: int = 8):
    B, H = 256, 32
    cu, idx = synthetic.equal_length_metadata(B, 1, device="cuda")
    pool = synthetic.state_pool(B, H, D, seed=5, device="cuda").half()
    elapsed = torch.zeros(B, dtype=torch.int32, device="cuda")
    toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=6)]
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B, max_seqlen=1)
    for _ in range(reps):
        F.infer_recurrent_fp16_forward_varlen(*toks, state_pool=pool, elapsed_state_pool=elapsed, cu_seqlens=cu,
                                              state_indices=idx, validated_metadata=ticket, max_seqlen=1)
        F.infer_recurrent_fp16_advance_i32(elapsed, 1)


def case_glue(reps: int = 2):
    B, T, C = 2, 4096, 4096
    gen = torch.Generator(device="cuda").manual_seed(7)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=gen).to(torch.bfloat16).requires_grad_()  # noqa: E731
    x, r, k, v, g = (rn(B, T, C) for _ in range(5))
    vecs = [rn(C) for _ in range(6)]
    r_k = rn(C // D, D)
    go = [torch.randn(B, T, C, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(6)]
    for _ in range(reps):
        outs = [F.pretrain_tmix_a_gate_bf16(vecs[0], x), F.pretrain_tmix_vres_gate_bf16(x, r, vecs[0], k),
                *F.pretrain_tmix_kk_pre_bf16(x, vecs[0], r, vecs[1]),
                F.pretrain_tmix_lnx_rkvres_xg_bf16(x, r, k, v, r_k, vecs[1], vecs[2], g)]
        torch.autograd.backward(outs, go[:len(outs)])
        torch.autograd.backward(F.pretrain_tmix_mix6_bf16(x, *vecs), go)


if __name__ == "__main__":
    cases = {"glue": case_glue, "chunk": case_chunk, "train": case_train, "train512": lambda: case_train(2, 8, 512, 64), "tmix": case_tmix, "decode": case_decode, "decode16": case_decode16}
    name = sys.argv[1] if len(sys.argv) > 1 else ""
    if name not in cases:
        raise SystemExit(__doc__)
    cases[name]()
    torch.cuda.synchronize()
    print(f"profile case {name}: done")
