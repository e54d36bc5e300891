"""Parity of the chunked (tensor-core) forward with the CPU oracle, the golden vectors and the recurrent kernel.

Tolerances: fp32 output within 2e-2 max-abs and final state within 1e-3 relative error of the float64 oracle
on identical 16-bit inputs; chunked and recurrent CUDA paths within the same bounds of each other.  The
reference's own criteria are checked too: relative RMSE <= 7e-3 (output) / 8e-3 (state) for the fp32-state
chunk family, 2e-2 for the bf16-state operator (tests/fixtures/tolerances-v1.json:13-26 of the reference),
allclose(atol=2e-3) on its RL case (tests/rl_infctx/wkv7/test.py:127-131 there).
"""
import pytest
import torch

from _util import load_golden, max_abs, rel_rmse

pytestmark = pytest.mark.gpu

TOKENS = ("r", "w", "k", "v", "a", "b")
Y_MAX_ABS = 2e-2
STATE_REL = 1e-3


def _state_rel(actual, expected):
    e = torch.as_tensor(expected).double()
    a = torch.as_tensor(actual).double().cpu()
    return float((a - e).norm() / e.norm().clamp_min(1e-30))


def test_golden_bf16_state_operator_ragged_tail():
    import flashrwkv_b200 as F

    g = load_golden("chunk_bf16")
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda().clone()
    before = pool.clone()
    y = F.infer_chunk_bf16_forward_varlen(*toks, state_pool=pool, cu_seqlens=g["cu_seqlens"].cuda(),
                                          state_indices=g["state_indices"].cuda(), chunk_size=8, scale=g["scale"])
    torch.cuda.synchronize()
    assert y.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16
    assert rel_rmse(y.float().cpu(), g["y"].float()) <= 2e-2
    assert rel_rmse(pool.float().cpu(), g["final_pool"].float()) <= 2e-2
    for slot in (1, 4):
        assert torch.equal(pool[slot], before[slot])
    with pytest.raises((ValueError, RuntimeError)):
        F.infer_chunk_bf16_forward_varlen(*toks, state_pool=pool, cu_seqlens=g["cu_seqlens"].cuda(),
                                          state_indices=torch.tensor([2, 2, 3], dtype=torch.int32, device="cuda"))


def test_golden_rl_fp16_new_pool_returned_input_untouched():
    import flashrwkv_b200 as F

    g = load_golden("rl_fp16")
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda()
    original = pool.clone()
    outs = {}
    for strategy in ("materialized", "recompute"):
        y, new_pool = F.rl_infctx_chunk_fp32io16(*toks, state_pool=pool, cu_seqlens=g["cu_seqlens"].cuda(),
                                                 state_indices=g["state_indices"].cuda(), chunk_size=16,
                                                 strategy=strategy, decay_bias=g["decay_bias"].cuda())
        torch.cuda.synchronize()
        assert y.dtype == torch.float16
        assert torch.allclose(y.float().cpu(), g["y"].float(), rtol=0.0, atol=2e-3)
        assert torch.allclose(new_pool.cpu(), g["final_pool"], rtol=0.0, atol=2e-3)
        assert rel_rmse(y.float().cpu(), g["y"].float()) <= 7e-3
        assert rel_rmse(new_pool.cpu(), g["final_pool"]) <= 8e-3
        outs[strategy] = (y, new_pool)
    assert torch.equal(outs["materialized"][0], outs["recompute"][0])
    assert torch.equal(pool, original)
    inactive = torch.tensor([0, 2], device="cuda")
    assert torch.equal(outs["recompute"][1].index_select(0, inactive), pool.index_select(0, inactive))
    with pytest.raises(ValueError, match="duplicates"):
        F.rl_infctx_chunk_fp32io16(*toks, state_pool=pool, cu_seqlens=g["cu_seqlens"].cuda(),
                                   state_indices=torch.tensor([1, 1], dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rl_wide_heads_vs_oracle(oracle, d, dtype):
    """Head sizes 128 / 256 of the RL operator (shapes and bounds of the reference's tests,
    tests/rl_infctx/wkv7/test.py:83-135 and :138-190): ragged lengths, scattered slots, decay bias, a 65-token tail."""
    import flashrwkv_b200 as F

    gen = torch.Generator().manual_seed(37 + d)
    for lengths, slots_of in (((2, 5), [3, 1]), ((65,), [1])):
        total, h = sum(lengths), 1
        toks = [(torch.randn(total, h, d, generator=gen) * 0.01).to(dtype) for _ in range(6)]
        pool = torch.randn(4, h, d, d, generator=gen) * 0.01
        cu = torch.tensor([0, *torch.tensor(lengths).cumsum(0).tolist()], dtype=torch.int32)
        idx = torch.tensor(slots_of, dtype=torch.int32)
        bias = (torch.randn(h, d, generator=gen) * 0.01).to(dtype)
        want = oracle.forward(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx, decay_bias=bias)
        d_pool = pool.cuda()
        for strategy in ("materialized", "recompute"):
            y, new_pool = F.rl_infctx_chunk_fp32io16(*[t.cuda() for t in toks], state_pool=d_pool, cu_seqlens=cu.cuda(),
                                                     state_indices=idx.cuda(), chunk_size=16, strategy=strategy,
                                                     decay_bias=bias.cuda())
            torch.cuda.synchronize()
            assert y.dtype == dtype and y.shape == toks[3].shape
            assert torch.allclose(y.float().cpu(), torch.as_tensor(want["y"]).float(), rtol=0.0, atol=2e-3)
            assert torch.allclose(new_pool.cpu(), torch.as_tensor(want["state_pool"]), rtol=0.0, atol=2e-3)
            untouched = [s for s in range(4) if s not in slots_of]
            assert torch.equal(new_pool[untouched].cpu(), pool[untouched])
            assert torch.equal(d_pool.cpu(), pool)


@pytest.mark.parametrize("path", [0, 1], ids=["build_scan", "fused"])
@pytest.mark.parametrize("lengths", [(512, 512), (1, 15, 16, 17, 65, 130, 64, 63)])
def test_chunked_vs_oracle_and_recurrent(oracle, lengths, path):
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    H, D = 3, 64
    N = sum(lengths)
    toks = synthetic.wkv7_inputs(N, H, D, seed=21 + len(lengths))
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    slots = torch.randperm(len(lengths) + 2)[: len(lengths)].to(torch.int32)
    pool0 = synthetic.state_pool(len(lengths) + 2, H, D, seed=9)
    bias = (torch.randn(H, D) * 0.2).to(torch.bfloat16)
    ref = oracle.forward(*toks, state_pool=pool0, cu_seqlens=cu, state_indices=slots, scale=0.7, decay_bias=bias)

    dtoks = [t.cuda() for t in toks]
    pool = pool0.cuda()
    y32 = torch.empty((N, H, D), device="cuda")
    meta = make_chunk_metadata(cu.cuda(), 64)
    sda = torch.full((N, H, D), float("nan"), device="cuda") if path == 1 else None
    y, boundary, flag = wkv7_chunk_forward(*dtoks, state=pool, chunk_metadata=meta, state_indices=slots.cuda(),
                                           scale=0.7, decay_bias=bias.cuda(), want_boundary=True, output_fp32=y32,
                                           state_dot_a=sda, path=path)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    if sda is not None:  # S_{t-1}^T a_t per token, the backward's saved tensor
        want = oracle.forward(*toks, state_pool=pool0, cu_seqlens=cu, state_indices=slots, decay_bias=bias,
                              want_state_dot_a=True)["state_dot_a"]
        assert rel_rmse(sda.cpu(), want) <= 2e-3
    assert max_abs(y32.cpu(), ref["y"]) <= Y_MAX_ABS
    assert rel_rmse(y.float().cpu(), ref["y"]) <= 7e-3
    assert _state_rel(pool, ref["state_pool"]) <= STATE_REL
    assert torch.equal(y, y32.to(y.dtype))
    # per-chunk boundary states against the oracle's
    ref_b = oracle.forward(*toks, state_pool=pool0, cu_seqlens=cu, state_indices=slots, scale=0.7, decay_bias=bias,
                           chunks=tuple(m.cpu() for m in meta))["boundary"]
    assert _state_rel(boundary, ref_b) <= STATE_REL
    # the recurrent kernel on the same inputs
    pool_r = pool0.cuda()
    y32_r = torch.empty_like(y32)
    F.infer_recurrent_fp32io16_forward_varlen(*dtoks, state_pool=pool_r, cu_seqlens=cu.cuda(),
                                              state_indices=slots.cuda(), scale=0.7, decay_bias=bias.cuda(),
                                              output_fp32=y32_r)
    torch.cuda.synchronize()
    assert max_abs(y32.cpu(), y32_r.cpu()) <= Y_MAX_ABS
    assert _state_rel(pool, pool_r.cpu()) <= STATE_REL
    # untouched slots stay bit-identical
    for slot in range(pool0.shape[0]):
        if slot not in slots.tolist():
            assert torch.equal(pool[slot].cpu(), pool0[slot])


@pytest.mark.parametrize("path", [0, 1], ids=["build_scan", "fused"])
def test_bad_metadata_status_fails_closed(path):
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    toks = [t.cuda() for t in synthetic.wkv7_inputs(70, 2, 64, seed=1)]
    cu = torch.tensor([0, 70], dtype=torch.int32, device="cuda")
    pool = synthetic.state_pool(1, 2, 64, seed=2, device="cuda")
    before = pool.clone()
    status = torch.tensor([4], dtype=torch.int32, device="cuda")
    y, _, _ = wkv7_chunk_forward(*toks, state=pool, chunk_metadata=make_chunk_metadata(cu), metadata_status=status,
                                 path=path)
    torch.cuda.synchronize()
    assert torch.isnan(y.float()).all()
    assert torch.equal(pool, before)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_and_two_kernel_forms_agree_many_pairs(oracle, dtype):
    """More (sequence, head) pairs than resident CTAs of a small grid would hold, ragged lengths, fp16 and bf16:
    the fused kernel against the build + scan pair and the oracle."""
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    H, D = 8, 64
    lengths = [64 * (1 + (i % 3)) + (i % 5) for i in range(48)]  # 384 pairs
    N = sum(lengths)
    toks = [t.to(dtype) for t in synthetic.wkv7_inputs(N, H, D, seed=77)]
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    pool0 = synthetic.state_pool(len(lengths), H, D, seed=78)
    dtoks = [t.cuda() for t in toks]
    meta = make_chunk_metadata(cu.cuda(), 64)
    outs = []
    for path in (0, 1):
        pool = pool0.cuda()
        y32 = torch.empty((N, H, D), device="cuda")
        _, _, flag = wkv7_chunk_forward(*dtoks, state=pool, chunk_metadata=meta, output_fp32=y32, path=path)
        torch.cuda.synchronize()
        assert int(flag.item()) == 0
        outs.append((y32.cpu(), pool.cpu()))
    ref = oracle.forward(*toks, state_pool=pool0, cu_seqlens=cu)
    for y32, pool in outs:
        assert max_abs(y32, ref["y"]) <= Y_MAX_ABS
        assert _state_rel(pool, ref["state_pool"]) <= STATE_REL
    assert max_abs(outs[0][0], outs[1][0]) <= Y_MAX_ABS


def test_reference_named_native_chunk_entries(oracle):
    """`_C.infer_chunk_bf16_forward_varlen` and `_C.rl_infctx_chunk_fp32io16_backward_replay` with the reference's
    argument order (csrc/sm120/tmix/wkv7/infer_chunk_bf16_forward_varlen.cpp:173-183 and
    csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_backward.cpp:102-135 there)."""
    from flashrwkv_b200 import _ext, synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    C = _ext.extension()
    g = load_golden("chunk_bf16")
    toks = [g[n].cuda() for n in TOKENS]
    pool = g["state_pool"].cuda().clone()
    y, same_pool = C.infer_chunk_bf16_forward_varlen(*toks, pool, g["cu_seqlens"].cuda(), g["state_indices"].cuda(), 8,
                                                    -1, g["scale"])
    torch.cuda.synchronize()
    assert same_pool.data_ptr() == pool.data_ptr()
    assert rel_rmse(y.float().cpu(), g["y"].float()) <= 2e-2
    assert rel_rmse(pool.float().cpu(), g["final_pool"].float()) <= 2e-2

    # replay stage: output and state_dot_a of every chunk from its boundary state
    H, D, lengths = 2, 64, (70, 16, 33)
    N = sum(lengths)
    toks = synthetic.wkv7_inputs(N, H, D, seed=91, dtype=torch.float16)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    pool0 = synthetic.state_pool(len(lengths), H, D, seed=92)
    bias = (torch.randn(H, D) * 0.1).to(torch.float16)
    meta = make_chunk_metadata(cu.cuda(), 32)
    dtoks = [t.cuda() for t in toks]
    _, boundary, _ = wkv7_chunk_forward(*dtoks, state=pool0.cuda(), chunk_metadata=meta, scale=0.6,
                                        decay_bias=bias.cuda(), want_boundary=True)
    out = torch.empty_like(dtoks[3])
    sda = torch.empty(N, H, D, device="cuda")
    C.rl_infctx_chunk_fp32io16_backward_replay(meta[1], meta[2], boundary, *dtoks, out, sda, 0.6, bias.cuda())
    torch.cuda.synchronize()
    want = oracle.forward(*toks, state_pool=pool0, cu_seqlens=cu, scale=0.6, decay_bias=bias, want_state_dot_a=True)
    assert torch.allclose(out.float().cpu(), torch.as_tensor(want["y"]).float(), rtol=0.0, atol=2e-2)
    assert rel_rmse(out.float().cpu(), want["y"]) <= 7e-3
    assert rel_rmse(sda.cpu(), want["state_dot_a"]) <= 2e-3
