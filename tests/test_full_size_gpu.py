"""Parity at the benchmark's full sizes, through properties that need no oracle run of that size.

The CPU oracle covers sizes it finishes in seconds (the other test files); here the four named configurations run
at full size and are checked through what the recurrence guarantees whatever the size:
  * two independent CUDA code paths agree (decode ring kernel vs register kernel; tensor-core chunk path vs
    recurrence),
  * the map (S0, v) -> (y, S_final) is linear for fixed r, w, k, a, b,
  * the backward is linear in the upstream gradient,
  * untouched state slots stay bit-identical and repeated runs are bit-identical.
Tolerances are the parity bars of the small-size tests (2e-2 max-abs on the fp32 output, 1e-3 relative on the state).
"""
import ctypes

import pytest
import torch

from _util import max_abs, rel_rmse

pytestmark = pytest.mark.gpu

D = 64


def _state_rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))


def test_cfg1_decode_ring_vs_register_kernel_and_linearity():
    """B=256, H=32 decode step: ring kernel (operator, max_seqlen=1) against the register kernel (C ABI call that
    does not declare the batch a decode batch), then linearity in (S0, v)."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import _ext, synthetic

    B, H = 256, 32
    toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=41)]
    cu, idx = (t.cuda() for t in synthetic.equal_length_metadata(B, 1))
    pool0 = synthetic.state_pool(B + 2, H, D, seed=42, device="cuda")  # two extra slots stay untouched
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B + 2, max_seqlen=1)

    def ring(tokens, pool):
        y32 = torch.empty(B, H, D, device="cuda")
        F.infer_recurrent_fp32io16_forward_varlen(*tokens, state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                  validated_metadata=ticket, max_seqlen=1, output_fp32=y32)
        return y32

    pool_a = pool0.clone()
    y_a = ring(toks, pool_a)
    pool_a2 = pool0.clone()
    y_a2 = ring(toks, pool_a2)  # the ticket alternates the traversal order between launches: same result
    assert torch.equal(y_a, y_a2) and torch.equal(pool_a, pool_a2)
    assert torch.equal(pool_a[B:], pool0[B:])

    lib = _ext.capi()
    pool_b = pool0.clone()
    y_b = torch.empty(B, H, D, device="cuda", dtype=torch.bfloat16)
    y32_b = torch.empty(B, H, D, device="cuda")
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.frwkv_wkv7_recurrent_fp32io16_forward_varlen(
        p(cu), p(idx), p(status), p(pool_b), *(p(t) for t in toks), None, p(y_b), p(y32_b), B, B, H, D, -1, 1,
        ctypes.c_float(1.0), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.frwkv_last_error()
    torch.cuda.synchronize()
    assert max_abs(y_a.cpu(), y32_b.cpu()) <= 1e-4  # same arithmetic, different data path
    assert _state_rel(pool_a.cpu(), pool_b.cpu()) <= 1e-6

    # linearity with the other five token tensors fixed: (S0a + S0b, v + v) -> y(S0a, v) + y(S0b, v); doubling v is
    # exact in bf16, the fp32 sum of the two pools is rounded once
    pool_c = synthetic.state_pool(B + 2, H, D, seed=43, device="cuda")
    v_twice = (toks[3].float() * 2).to(torch.bfloat16)
    assert torch.equal(v_twice.float(), toks[3].float() * 2)
    p1, p2, p12 = pool0.clone(), pool_c.clone(), pool0 + pool_c
    y1, y2 = ring(toks, p1), ring(toks, p2)
    y12 = ring([toks[0], toks[1], toks[2], v_twice, toks[4], toks[5]], p12)
    torch.cuda.synchronize()
    assert float((y12 - (y1 + y2)).abs().max()) <= 1e-3
    assert _state_rel((p1 + p2)[:B].cpu(), p12[:B].cpu()) <= 1e-5


def test_cfg2_chunked_prefill_vs_recurrence_full_size():
    """B=8, T=4096, H=32: the tensor-core chunk path against the fp32 recurrence on the same inputs."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    B, T, H = 8, 4096, 32
    toks = [t.cuda() for t in synthetic.wkv7_inputs(B * T, H, D, seed=44)]
    cu, idx = (t.cuda() for t in synthetic.equal_length_metadata(B, T))
    pool0 = synthetic.state_pool(B, H, D, seed=45, device="cuda")
    pool_c, pool_r = pool0.clone(), pool0.clone()
    y32_c = torch.empty(B * T, H, D, device="cuda")
    y32_r = torch.empty(B * T, H, D, device="cuda")
    out = wkv7_chunk_forward(*toks, state=pool_c, chunk_metadata=make_chunk_metadata(cu, 64), output_fp32=y32_c)
    F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool_r, cu_seqlens=cu, state_indices=idx,
                                              output_fp32=y32_r)
    torch.cuda.synchronize()
    assert int(out[2].item()) == 0
    assert torch.isfinite(y32_c).all()
    assert float((y32_c - y32_r).abs().max()) <= 2e-2
    assert rel_rmse(y32_c.cpu(), y32_r.cpu()) <= 2e-3
    assert _state_rel(pool_c.cpu(), pool_r.cpu()) <= 1e-3
    # the 16-bit output is the rounded fp32 output
    assert torch.equal(out[0], y32_c.to(torch.bfloat16))


def test_cfg3_training_backward_is_linear_in_upstream_gradient():
    """B=8, T=4096, H=64 forward + backward: for all seven gradients grads(dy1 + dy2) = grads(dy1) + grads(dy2) (the
    token gradients are rounded to bf16 once, hence the tolerance), and a repeated backward is bit-identical."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata

    B, T, H = 8, 4096, 64
    toks = [t.cuda().requires_grad_() for t in synthetic.wkv7_inputs(B * T, H, D, seed=46)]
    S0 = synthetic.state_pool(B, H, D, seed=47, device="cuda").requires_grad_()
    cu, _ = synthetic.equal_length_metadata(B, T, device="cuda")
    meta = make_chunk_metadata(cu, 64)
    gen = torch.Generator(device="cuda").manual_seed(48)
    dy1 = torch.randn(B * T, H, D, device="cuda", generator=gen).to(torch.bfloat16)
    dy2 = torch.randn(B * T, H, D, device="cuda", generator=gen).to(torch.bfloat16)
    dy12 = (dy1.float() + dy2.float()).to(torch.bfloat16)
    out = F.statetune_recurrent_fp32io16(S0, *meta, *toks)

    def grads(dy):  # all seven gradients: r, decay logits, k, v, a, b and the initial state
        g = torch.autograd.grad(out[0], [S0, *toks], dy, retain_graph=True)
        return [t.float() for t in g]

    names = ("dS0", "dr", "dw", "dk", "dv", "da", "db")
    g1, g2, g12 = grads(dy1), grads(dy2), grads(dy12)
    for a, b, c, name in zip(g1, g2, g12, names):
        assert torch.isfinite(c).all(), name
        assert rel_rmse(a + b, c) <= 1.5e-2, name
    del g1, g2
    for a, b, name in zip(g12, grads(dy12), names):
        assert torch.equal(a, b), name
    # the last 256 tokens of two sequences against the oracle's float64 backward is what tests/test_training_gpu.py
    # does at T = 256; here the whole-length run only has to agree with itself and be linear
