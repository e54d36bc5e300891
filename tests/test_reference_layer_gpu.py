"""The reference's own, unmodified Python package on top of this build's native module.

`baseline/_ref/flashrwkv2` is the reference project installed as it ships (its Python operator layer: argument
validation, output allocation, autograd wrappers).  Here its native module `flashrwkv2._C` is this build's `_C`, and
its dense pretraining operator finds `torch.ops.rwkv7_clampw_v3` registered by the same module.  Every hot-path
operator is then called through the reference's wrappers and checked against the golden vectors made from the
reference's test oracles: what passes here is what a user of the reference gets after swapping the native module.

Skipped when the reference package is not installed next to the repository's sources.
"""
from __future__ import annotations

import importlib
import sys
from pathlib import Path

import pytest
import torch

from _util import load_golden, max_abs, rel_rmse

pytestmark = pytest.mark.gpu

REF_ROOT = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
TOKENS = ("r", "w", "k", "v", "a", "b")


@pytest.fixture(scope="module")
def ref():
    if not (REF_ROOT / "flashrwkv2" / "__init__.py").exists():
        pytest.skip("the reference package is not installed under baseline/_ref")
    from flashrwkv_b200._ext import extension

    native = extension()
    saved_path = list(sys.path)
    sys.modules["flashrwkv2._C"] = native  # the reference's `from . import _C` resolves to this build
    sys.path.insert(0, str(REF_ROOT))
    try:
        module = importlib.import_module("flashrwkv2")
        module._C = native
        assert Path(module.__file__).resolve().is_relative_to(REF_ROOT)
        yield module
    finally:
        sys.path[:] = saved_path
        for name in [n for n in sys.modules if n == "flashrwkv2" or n.startswith("flashrwkv2.")]:
            del sys.modules[name]


def test_native_names_the_reference_calls_are_all_exported(ref):
    import re

    native = ref._C
    wanted = set()
    for path in (REF_ROOT / "flashrwkv2" / "tmix").rglob("*.py"):
        wanted |= set(re.findall(r"_extension\(\)\s*\.\s*([A-Za-z0-9_]+)", path.read_text()))
    for path in (REF_ROOT / "flashrwkv2" / "rl_infctx").rglob("*.py"):
        wanted |= set(re.findall(r"(?:_extension\(\)|extension)\s*\.\s*([A-Za-z0-9_]+)\(", path.read_text()))
    assert len(wanted) >= 40
    missing = sorted(n for n in wanted if not hasattr(native, n))
    assert not missing, missing
    assert hasattr(torch.ops.rwkv7_clampw_v3, "forward") and hasattr(torch.ops.rwkv7_clampw_v3, "backward")


def test_recurrent_fp32_state_through_reference_wrapper(ref):
    g = load_golden("recurrent_ragged")
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda().clone()
    cu, idx = g["cu_seqlens"].cuda(), g["state_indices"].cuda()
    y = ref.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                    scale=g["scale"], decay_bias=g["decay_bias"].cuda())
    assert y.dtype == torch.bfloat16
    assert rel_rmse(y.float().cpu(), g["y"].float()) <= 8e-3
    assert rel_rmse(pool.cpu(), g["final_pool"]) <= 8e-3
    # the prepared-metadata ticket of the reference's API, reused across launches
    ticket = ref.prepare_recurrent_metadata(cu, idx, total_tokens=toks[0].shape[0], state_pool_size=pool.shape[0])
    pool2 = g["state_pool"].cuda().clone()
    y2 = ref.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool2, cu_seqlens=cu, state_indices=idx,
                                                     scale=g["scale"], decay_bias=g["decay_bias"].cuda(),
                                                     validated_metadata=ticket)
    assert torch.equal(y, y2) and torch.equal(pool, pool2)


def test_recurrent_fp16_state_through_reference_wrapper(ref):
    g = load_golden("recurrent_fp16state")
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda().clone()
    elapsed = g["elapsed_state_pool"].cuda().clone()
    y = ref.infer_recurrent_fp16_forward_varlen(*toks, state_pool=pool, elapsed_state_pool=elapsed,
                                                cu_seqlens=g["cu_seqlens"].cuda(),
                                                state_indices=g["state_indices"].cuda(), scale=g["scale"],
                                                decay_bias=g["decay_bias"].cuda())
    assert y.dtype == torch.float16
    assert rel_rmse(y.float().cpu(), g["y"].float()) <= 8e-3
    assert rel_rmse(pool.float().cpu(), g["final_pool"].float()) <= 8e-3


def test_chunk_bf16_through_reference_wrapper(ref):
    g = load_golden("chunk_bf16")
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda().clone()
    y = ref.infer_chunk_bf16_forward_varlen(*toks, state_pool=pool, cu_seqlens=g["cu_seqlens"].cuda(),
                                            state_indices=g["state_indices"].cuda(), chunk_size=16, scale=g["scale"])
    assert y.dtype == torch.bfloat16
    assert rel_rmse(y.float().cpu(), g["y"].float()) <= 2e-2
    assert rel_rmse(pool.float().cpu(), g["final_pool"].float()) <= 2e-2


def test_rl_infctx_chunk_through_reference_wrapper(ref):
    g = load_golden("rl_fp16")
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda()
    before = pool.clone()
    for strategy in ("materialized", "recompute"):
        y, new_pool = ref.rl_infctx_chunk_fp32io16(*toks, state_pool=pool, cu_seqlens=g["cu_seqlens"].cuda(),
                                                   state_indices=g["state_indices"].cuda(), chunk_size=16,
                                                   strategy=strategy, decay_bias=g["decay_bias"].cuda())
        assert torch.allclose(y.float().cpu(), g["y"].float(), rtol=0.0, atol=2e-3)
        assert torch.allclose(new_pool.cpu(), g["final_pool"], rtol=0.0, atol=2e-3)
    assert torch.equal(pool, before)


def test_statetune_through_reference_autograd(ref):
    g = load_golden("statetune")
    S0 = g["S0"].cuda().requires_grad_()
    toks = [g[n].cuda().requires_grad_() for n in TOKENS]
    out = ref.statetune_recurrent_fp32io16(S0, g["seq_chunk_offsets"].cuda(), g["chunk_starts"].cuda(),
                                           g["chunk_ends"].cuda(), *toks, scale=g["scale"])
    for got, name in zip(out, ("y", "final_state", "boundary", "state_dot_a")):
        assert torch.allclose(got.float().cpu(), g[name].float(), atol=3e-4, rtol=3e-4), name
    (out[0].float().square().sum() + out[1].square().sum()).backward()
    for t, name in zip([S0, *toks], ("dS0", "dr", "dw", "dk", "dv", "da", "db")):
        assert torch.allclose(t.grad.float().cpu(), g[name], atol=3e-4, rtol=3e-3), name


def test_pretrain_through_reference_autograd_and_op_library(ref, oracle):
    g = load_golden("pretrain")
    vals = [g[n].cuda().requires_grad_() for n in TOKENS]
    y = ref.pretrain_recurrent_bf16(*vals)
    assert torch.allclose(y.float().cpu(), g["y"], atol=0.02, rtol=0.02)
    y.backward(g["dy"].cuda())
    for t, name in zip(vals, ("dr", "dw", "dk", "dv", "da", "db")):
        assert torch.allclose(t.grad.float().cpu(), g[name], atol=0.03, rtol=0.05), name
    # the saved tensors of the op library itself: the state after every 16 tokens [B,H,T/16,key,value] and sa
    B, T, C = vals[0].shape
    H = C // 64
    four = [v.detach().view(B, T, H, 64) for v in vals]
    out = torch.empty_like(four[3])
    s = torch.full((B, H, T // 16, 64, 64), float("nan"), device="cuda")
    sa = torch.full((B, T, H, 64), float("nan"), device="cuda")
    torch.ops.rwkv7_clampw_v3.forward(*four, out, s, sa, 64)
    assert torch.equal(out.view(B, T, C), y.detach())
    G = T // 16
    cs = torch.arange(G, dtype=torch.int32) * 16
    for bi in range(B):
        packed = [t[bi].float().cpu() for t in four]
        want = oracle.forward(*packed, state_pool=torch.zeros(1, H, 64, 64),
                              cu_seqlens=torch.tensor([0, T], dtype=torch.int32),
                              chunks=(torch.tensor([0, G], dtype=torch.int32), cs, cs + 16), want_state_dot_a=True)
        assert max_abs(sa[bi].cpu(), want["state_dot_a"]) <= 3e-4
        for c in range(G):
            after = want["boundary"][c + 1] if c + 1 < G else want["state_pool"][0]
            assert max_abs(s[bi, :, c].cpu(), after) <= 3e-4


@pytest.mark.parametrize("head_size", [128, 256])
def test_wide_head_training_through_reference_wrappers(ref, head_size):
    """Head sizes 128 / 256: the reference's pretrain and StateTune autograd wrappers over this module give the
    bits of this package's own wrappers (which tests/test_training_gpu.py checks against the oracle)."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata

    B, T, H, D = 1, 48, 1, head_size
    gen = torch.Generator().manual_seed(D)
    base = [(torch.randn(B, T, H * D, generator=gen) * sc).to(torch.bfloat16).cuda()
            for sc in (0.12, 2.0, 0.1, 0.1, 0.1, 0.1)]
    dy = torch.randn(B, T, H * D, generator=gen).to(torch.bfloat16).cuda()
    grads = []
    for impl in (ref, F):
        vals = [t.clone().requires_grad_() for t in base]
        y = impl.pretrain_recurrent_bf16(*vals, head_size=D)
        y.backward(dy)
        grads.append([y.detach()] + [v.grad for v in vals])
    for a, b in zip(*grads):
        assert torch.isfinite(a).all() and torch.equal(a, b)
    lengths = (20, 33)
    cu = torch.tensor([0, 20, 53], dtype=torch.int32, device="cuda")
    meta = make_chunk_metadata(cu, 32)
    toks = [t.cuda() for t in synthetic.wkv7_inputs(sum(lengths), H, D, seed=D)]
    S0 = synthetic.state_pool(2, H, D, seed=2, device="cuda")
    outs = []
    for impl in (ref, F):
        s0 = S0.clone().requires_grad_()
        leaves = [t.clone().requires_grad_() for t in toks]
        res = impl.statetune_recurrent_fp32io16(s0, *meta, *leaves, scale=0.9)
        (res[0].float().sum() + res[1].sum()).backward()
        outs.append([r.detach() for r in res] + [s0.grad] + [t.grad for t in leaves])
    for a, b in zip(*outs):
        assert torch.isfinite(a).all() and torch.equal(a, b)


def test_projections_through_reference_wrappers_both_layouts(ref):
    gen = torch.Generator().manual_seed(11)
    M, C, R = 9, 256, 64
    x = (torch.randn(M, C, generator=gen)).half().cuda()
    w1 = (torch.randn(R, C, generator=gen) * 0.05).half().cuda()  # original layout [N,K]
    w2 = (torch.randn(C, R, generator=gen) * 0.05).half().cuda()
    want1 = x.float() @ w1.float().T
    got_t = ref.infer_tmix_linear_rank_in_forward_varlen(x, weight_t=w1)
    got_rt = ref.infer_tmix_linear_rank_in_forward_varlen(x, weight=w1.t().contiguous())
    assert rel_rmse(got_t.float().cpu(), want1.cpu()) <= 2e-3
    assert rel_rmse(got_rt.float().cpu(), want1.cpu()) <= 2e-3
    want2 = torch.tanh(got_t.float()) @ w2.float().T
    got2 = ref.infer_tmix_linear_rank_out_tanh_forward_varlen(got_t, weight_t=w2)
    assert rel_rmse(got2.float().cpu(), want2.cpu()) <= 2e-3
    W = (torch.randn(C, C, generator=gen) * 0.05).half().cuda()
    dense = ref.infer_tmix_linear_forward_varlen(x, W)
    dense_rt = ref.infer_tmix_linear_forward_varlen(x, W.t().contiguous(), weight_is_transposed=True)
    want = (x.float() @ W.float().T).cpu()
    assert rel_rmse(dense.float().cpu(), want) <= 2e-3
    assert rel_rmse(dense_rt.float().cpu(), want) <= 2e-3


def test_mix6_and_per_head_glue_through_reference_wrappers(ref):
    g = load_golden("tmix_mix6")
    x, pool = g["x"].cuda(), g["shift_pool"].cuda().clone()
    cu, idx = g["cu_seqlens"].cuda(), g["state_indices"].cuda()
    outs = ref.infer_tmix_mix6_forward_varlen(x, *g["mix"].cuda().unbind(0), shift_state_pool=pool, cu_seqlens=cu,
                                              state_indices=idx)
    for j in range(6):
        assert torch.allclose(outs[j].float().cpu(), g["out"][j], atol=0.01, rtol=0.01)
    assert torch.equal(pool.cpu(), g["shift_after"])
    g = load_golden("tmix_kk_a_gate")
    outs = ref.infer_tmix_kk_a_gate_forward_varlen(*(g[n].cuda() for n in ("k", "k_k", "a0", "a12", "k_a")))
    for o, name in zip(outs, ("new_k", "neg_kk", "kka")):
        assert rel_rmse(o.float().cpu(), g[name]) <= 2e-3
    g = load_golden("tmix_lnx")
    out = ref.infer_tmix_lnx_rkvres_xg_forward_varlen(*(g[n].cuda() for n in ("x", "r", "k", "v", "r_k", "weight",
                                                                              "bias", "g")))
    assert rel_rmse(out.float().cpu(), g["out"]) <= 2e-3
    g = load_golden("tmix_vres")
    out = ref.infer_tmix_vres_gate_forward_varlen(*(g[n].cuda() for n in ("v", "v_first", "v0", "v12")))
    assert rel_rmse(out.float().cpu(), g["out"]) <= 2e-3
