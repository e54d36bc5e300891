"""Parity of the fp16-state recurrence (public operator -> C ABI -> CUDA) with the CPU oracle and the golden
vectors of the reference's own fp16 oracle.

Tolerance: the reference's gate for this path, relative RMSE <= 3e-3 for output and state
(tests/fixtures/tolerances-v1.json:27-29 of the reference).  The kernel follows the same rounding points
(fp16 retention increment with dither, one fp16 rounding of the new state, output from the rounded state), so the
state is additionally required to be bit-identical to the oracle's on all but a small fraction of values.
"""
import numpy as np
import pytest
import torch

from _util import load_golden, rel_rmse

pytestmark = pytest.mark.gpu

TOKENS = ("r", "w", "k", "v", "a", "b")
REF_RMSE = 3e-3


def _mismatch(actual: torch.Tensor, expected: torch.Tensor):
    """Fraction of fp16 values that differ at all, and the largest difference relative to the largest value.
    (A value that differs was a rounding tie broken the other way by the summation order of S^T a; values left
    near zero by cancellation may then differ by several of their own ulps, hence the absolute measure.)"""
    a, e = actual.float().cpu(), expected.float().cpu()
    return float((a != e).float().mean()), float((a - e).abs().max() / e.abs().max())


@pytest.mark.parametrize("name", ["recurrent_fp16state", "recurrent_fp16state_d128"])
def test_golden_vectors_from_reference_fp16_oracle(name):
    import flashrwkv_b200 as F

    g = load_golden(name)
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda().clone()
    elapsed = g["elapsed_state_pool"].cuda()
    y = F.infer_recurrent_fp16_forward_varlen(*toks, state_pool=pool, elapsed_state_pool=elapsed,
                                              cu_seqlens=g["cu_seqlens"].cuda(),
                                              state_indices=g["state_indices"].cuda(), scale=g["scale"],
                                              decay_bias=g["decay_bias"].cuda())
    torch.cuda.synchronize()
    assert y.dtype == torch.float16 and pool.dtype == torch.float16
    assert rel_rmse(y.float().cpu(), g["y"].float()) <= REF_RMSE
    assert rel_rmse(pool.float().cpu(), g["final_pool"].float()) <= REF_RMSE
    frac, worst = _mismatch(pool, g["final_pool"])
    assert frac < 5e-3 and worst <= 1e-3
    active = set(g["state_indices"].tolist())
    untouched = [s for s in range(pool.shape[0]) if s not in active]
    assert torch.equal(pool[untouched].cpu(), g["state_pool"][untouched])
    assert torch.equal(elapsed.cpu(), g["elapsed_state_pool"])  # read, never advanced


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H", [(64, 32), (40, 32), (3, 2)])
def test_decode_steps_vs_oracle(oracle, dtype, B, H):
    """Consecutive decode steps (one token per sequence) with the counters advanced in between; B*H >= 1024 runs the
    bulk-copy ring kernel, smaller batches the register kernel."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    D, slots = 64, B + 3
    gen = torch.Generator().manual_seed(B * 131 + H)
    pool = (torch.randn(slots, H, D, D, generator=gen) * 0.1).half()
    elapsed = torch.randint(0, 1 << 20, (slots,), generator=gen, dtype=torch.int32)
    idx = torch.randperm(slots, generator=gen)[:B].int()
    cu = torch.arange(B + 1, dtype=torch.int32)
    bias = (torch.randn(H, D, generator=gen) * 0.2).to(dtype)
    d_pool, d_elapsed, d_cu, d_idx = pool.cuda(), elapsed.cuda(), cu.cuda(), idx.cuda()
    ticket = F.prepare_recurrent_metadata(d_cu, d_idx, total_tokens=B, state_pool_size=slots, max_seqlen=1)
    ref_pool, ref_elapsed = pool.clone(), elapsed.clone()
    for step in range(3):
        toks = [t.to(dtype) for t in synthetic.wkv7_inputs(B, H, D, seed=500 + step, dtype=torch.float32)]
        y = F.infer_recurrent_fp16_forward_varlen(*[t.cuda() for t in toks], state_pool=d_pool,
                                                  elapsed_state_pool=d_elapsed, cu_seqlens=d_cu, state_indices=d_idx,
                                                  decay_bias=bias.cuda(), max_seqlen=1, validated_metadata=ticket)
        F.infer_recurrent_fp16_advance_i32_varlen(d_elapsed, d_cu, d_idx, total_tokens=B, validated_metadata=ticket)
        out = oracle.forward_fp16(*toks, state_pool=ref_pool, elapsed_state_pool=ref_elapsed, cu_seqlens=cu,
                                  state_indices=idx, decay_bias=bias)
        ref_pool = torch.from_numpy(out["state_pool"])
        ref_elapsed[idx.long()] += 1
        torch.cuda.synchronize()
        assert y.dtype == dtype
        assert rel_rmse(y.float().cpu(), out["y"]) <= REF_RMSE, f"step {step}"
        assert rel_rmse(d_pool.float().cpu(), ref_pool.float()) <= REF_RMSE, f"step {step}"
    frac, worst = _mismatch(d_pool, ref_pool)
    assert frac < 5e-3 and worst <= 1e-3
    assert torch.equal(d_elapsed.cpu(), ref_elapsed)
    untouched = [s for s in range(slots) if s not in set(idx.tolist())]
    assert torch.equal(d_pool[untouched].cpu(), pool[untouched])


def test_ragged_sequences_vs_oracle(oracle):
    import flashrwkv_b200 as F

    D, H, lengths, slots = 64, 3, (1, 15, 16, 17, 65, 2), 9
    N = sum(lengths)
    gen = torch.Generator().manual_seed(77)
    rnd = lambda s: (torch.randn(N, H, D, generator=gen) * s).half()  # noqa: E731
    toks = [rnd(0.12), rnd(3.5), rnd(0.06), rnd(0.06), rnd(0.06), rnd(0.06)]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
    idx = torch.tensor([5, 0, 7, 2, 4, 8], dtype=torch.int32)
    pool = (torch.randn(slots, H, D, D, generator=gen) * 0.03).half()
    elapsed = (torch.arange(slots, dtype=torch.int32) * 11)
    d_pool = pool.cuda()
    y = F.infer_recurrent_fp16_forward_varlen(*[t.cuda() for t in toks], state_pool=d_pool,
                                              elapsed_state_pool=elapsed.cuda(), cu_seqlens=cu.cuda(),
                                              state_indices=idx.cuda(), scale=0.5)
    out = oracle.forward_fp16(*toks, state_pool=pool, elapsed_state_pool=elapsed, cu_seqlens=cu, state_indices=idx,
                              scale=0.5)
    torch.cuda.synchronize()
    assert rel_rmse(y.float().cpu(), out["y"]) <= REF_RMSE
    assert rel_rmse(d_pool.float().cpu(), torch.from_numpy(out["state_pool"]).float()) <= REF_RMSE


@pytest.mark.parametrize("head_size", [128, 256])
@pytest.mark.parametrize("lengths", [(1,), (1, 2, 4), (8, 8), (33, 1, 7)])
def test_wide_heads_vs_oracle(oracle, head_size, lengths):
    """Head sizes 128 and 256 (the reference's fp16 family test runs these, tests/tmix/wkv7/test.py:1003-1060):
    decay bias, a scale, scattered slots, non-zero elapsed counters; untouched slots stay bit-identical."""
    import flashrwkv_b200 as F

    D, H, slots = head_size, 2, len(lengths) + 2
    N = sum(lengths)
    gen = torch.Generator().manual_seed(500 + head_size + N)
    rnd = lambda s: (torch.randn(N, H, D, generator=gen) * s).half()  # noqa: E731
    toks = [rnd(0.1), rnd(3.0), rnd(0.05), rnd(0.05), rnd(0.05), rnd(0.05)]
    bias = (torch.randn(H, D, generator=gen) * 0.5).half()
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
    idx = torch.randperm(slots, generator=gen)[:len(lengths)].to(torch.int32)
    pool = (torch.randn(slots, H, D, D, generator=gen) * 0.03).half()
    elapsed = torch.arange(slots, dtype=torch.int32) * 7 + 3
    d_pool, d_elapsed = pool.cuda(), elapsed.cuda()
    y = F.infer_recurrent_fp16_forward_varlen(*[t.cuda() for t in toks], state_pool=d_pool,
                                              elapsed_state_pool=d_elapsed, cu_seqlens=cu.cuda(),
                                              state_indices=idx.cuda(), scale=0.5, decay_bias=bias.cuda())
    out = oracle.forward_fp16(*toks, state_pool=pool, elapsed_state_pool=elapsed, cu_seqlens=cu, state_indices=idx,
                              scale=0.5, decay_bias=bias)
    torch.cuda.synchronize()
    want_pool = torch.from_numpy(out["state_pool"])
    assert torch.isfinite(y.float()).all()
    assert rel_rmse(y.float().cpu(), out["y"]) <= REF_RMSE
    assert rel_rmse(d_pool.float().cpu(), want_pool.float()) <= REF_RMSE
    frac, worst = _mismatch(d_pool, want_pool)
    assert frac <= 5e-3 and worst <= 2e-3, (frac, worst)
    untouched = [i for i in range(slots) if i not in set(idx.tolist())]
    assert torch.equal(d_pool[untouched].cpu(), pool[untouched])
    assert torch.equal(d_elapsed.cpu(), elapsed)  # the counters are read only


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_add_vec_helper_is_the_rounded_fp32_sum(dtype):
    """Shapes of the reference's test (tests/tmix/wkv7/test.py:131-138) plus an even channel count that is not a
    multiple of 8; bit-exact."""
    import flashrwkv_b200 as F

    for rows, channels in ((3, 8), (17, 4096), (5, 70)):
        x = torch.randn(rows, channels, device="cuda").to(dtype)
        vec = torch.randn(channels, device="cuda").to(dtype)
        out = F.infer_recurrent_add_vec_forward_varlen(x, vec)
        assert torch.equal(out, (x.float() + vec.float()).to(dtype))
    with pytest.raises(ValueError, match="even C"):
        F.infer_recurrent_add_vec_forward_varlen(x[:, :69].contiguous(), vec[:69].contiguous())


def test_elapsed_counter_operators_and_fail_closed():
    import flashrwkv_b200 as F

    e = torch.tensor([2, 7, 11], device="cuda", dtype=torch.int32)
    F.infer_recurrent_fp16_advance_i32(e, 5)
    assert e.tolist() == [7, 12, 16]
    e = torch.tensor([2, 5, 7, 11], device="cuda", dtype=torch.int32)
    cu = torch.tensor([0, 3, 4], device="cuda", dtype=torch.int32)
    idx = torch.tensor([2, 0], device="cuda", dtype=torch.int32)
    F.infer_recurrent_fp16_advance_i32_varlen(e, cu, idx, total_tokens=4)
    assert e.tolist() == [3, 5, 10, 11]
    with pytest.raises(TypeError):
        F.infer_recurrent_fp16_advance_i32(e.float(), 1)
    with pytest.raises(TypeError):
        F.infer_recurrent_fp16_advance_i32(e, 1.5)
    # duplicate slots: prepare refuses; the low-level call with a bad status word leaves everything untouched
    bad = torch.tensor([1, 1], device="cuda", dtype=torch.int32)
    with pytest.raises((RuntimeError, ValueError)):
        F.infer_recurrent_fp16_advance_i32_varlen(e, cu, bad, total_tokens=4)
    assert e.tolist() == [3, 5, 10, 11]
    # wrong state dtype / elapsed shape are refused before any launch
    toks = [torch.zeros(4, 1, 64, device="cuda", dtype=torch.float16) for _ in range(6)]
    with pytest.raises(TypeError, match="float16"):
        F.infer_recurrent_fp16_forward_varlen(*toks, state_pool=torch.zeros(4, 1, 64, 64, device="cuda"),
                                              elapsed_state_pool=e, cu_seqlens=cu, state_indices=idx)
    with pytest.raises(ValueError, match="state_pool_slots"):
        F.infer_recurrent_fp16_forward_varlen(*toks, state_pool=torch.zeros(5, 1, 64, 64, device="cuda").half(),
                                              elapsed_state_pool=e, cu_seqlens=cu, state_indices=idx)
