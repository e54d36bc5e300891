"""Training path: StateTune and dense pretraining forward outputs and gradients against the golden vectors
(the reference's oracles + autograd) and, at larger sizes, the CPU oracle's backward.

Tolerances are the reference's: StateTune outputs allclose(3e-4, 3e-4), gradients allclose(atol 3e-4, rtol 3e-3)
(tests/tmix/wkv7/statetune/test.py:107,123); pretraining forward allclose(0.02, 0.02), gradients
allclose(atol 0.03, rtol 0.05) (tests/tmix/wkv7/pretrain/test.py:104,126-128); plus relative RMSE <= 8e-3 on
gradients (tests/fixtures/tolerances-v1.json:13-17).
"""
import pytest
import torch

from _util import load_golden, max_abs, rel_rmse

pytestmark = pytest.mark.gpu
TOKENS = ("r", "w", "k", "v", "a", "b")


def test_golden_statetune_outputs_and_seven_gradients():
    import flashrwkv_b200 as F

    g = load_golden("statetune")
    S0 = g["S0"].cuda().requires_grad_()
    toks = [g[n].cuda().requires_grad_() for n in TOKENS]
    before = S0.detach().clone()
    out = F.statetune_recurrent_fp32io16(S0, g["seq_chunk_offsets"].cuda(), g["chunk_starts"].cuda(),
                                         g["chunk_ends"].cuda(), *toks, scale=g["scale"])
    for got, name in zip(out, ("y", "final_state", "boundary", "state_dot_a")):
        assert torch.allclose(got.float().cpu(), g[name].float(), atol=3e-4, rtol=3e-4), name
    (out[0].float().square().sum() + out[1].square().sum()).backward()
    for t, name in zip([S0, *toks], ("dS0", "dr", "dw", "dk", "dv", "da", "db")):
        assert torch.isfinite(t.grad).all()
        assert torch.allclose(t.grad.float().cpu(), g[name], atol=3e-4, rtol=3e-3), name
    assert torch.equal(S0.detach(), before)


def test_golden_pretrain_forward_and_gradients():
    import flashrwkv_b200 as F

    g = load_golden("pretrain")
    vals = [g[n].cuda().requires_grad_() for n in TOKENS]
    y = F.pretrain_recurrent_bf16(*vals)
    assert y.shape == vals[0].shape and y.dtype == torch.bfloat16
    assert torch.allclose(y.float().cpu(), g["y"], atol=0.02, rtol=0.02)
    assert torch.equal(y, F.pretrain_recurrent_bf16(*vals))
    y.backward(g["dy"].cuda())
    for t, name in zip(vals, ("dr", "dw", "dk", "dv", "da", "db")):
        assert torch.isfinite(t.grad).all()
        assert torch.allclose(t.grad.float().cpu(), g[name], atol=0.03, rtol=0.05), name
    with pytest.raises(ValueError, match="divisible by the canonical chunk length 16"):
        F.pretrain_recurrent_bf16(*(v[:, :17].contiguous() for v in vals))
    with pytest.raises(TypeError, match="bfloat16"):
        F.pretrain_recurrent_bf16(*(v.half() for v in vals))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("lengths", [(256, 256), (1, 17, 64, 100, 130)])
def test_gradients_vs_oracle_backward(oracle, lengths, dtype):
    """B200 gradients against the oracle's float64 backward at T up to 256, ragged chunking, non-zero S0,
    upstream gradients on both the output and the final state; both 16-bit token types."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata

    H, D, B = 2, 64, len(lengths)
    N = sum(lengths)
    toks = synthetic.wkv7_inputs(N, H, D, seed=31 + B, dtype=dtype)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    S0 = synthetic.state_pool(B, H, D, seed=5)
    gen = torch.Generator().manual_seed(8)
    dy = torch.randn(N, H, D, generator=gen).to(dtype)
    dSf = torch.randn(B, H, D, D, generator=gen) * 0.1
    want = oracle.backward(*toks, initial_state=S0, cu_seqlens=cu, grad_output=dy, grad_final_state=dSf, scale=0.8)
    dS0 = S0.cuda().requires_grad_()
    dtoks = [t.cuda().requires_grad_() for t in toks]
    meta = make_chunk_metadata(cu.cuda(), 64)
    out = F.statetune_recurrent_fp32io16(dS0, *meta, *dtoks, scale=0.8)
    torch.autograd.backward([out[0], out[1]], [dy.cuda(), dSf.cuda()])
    names = ("r", "decay_logits", "k", "v", "a", "b")
    for t, name in zip(dtoks, names):
        assert rel_rmse(t.grad.float().cpu(), want[name]) <= 8e-3, name
    assert rel_rmse(dS0.grad.cpu(), want["initial_state"]) <= 8e-3


def test_reference_named_native_statetune_entries_match_golden():
    """`_C.statetune_recurrent_fp32io16_forward` / `_backward` with the reference's argument order
    (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_{forward,backward}.cpp there): in-place final state, outputs and
    gradients written into caller tensors, optional gradients skipped."""
    from flashrwkv_b200 import _ext

    C = _ext.extension()
    g = load_golden("statetune")
    toks = [g[n].cuda() for n in TOKENS]
    sco, cs, ce = (g[n].cuda() for n in ("seq_chunk_offsets", "chunk_starts", "chunk_ends"))
    state = g["S0"].cuda().clone()
    y = torch.empty_like(toks[3])
    boundary = torch.empty(cs.numel(), state.shape[1], 64, 64, device="cuda")
    sda = torch.empty(toks[0].shape, device="cuda")
    C.statetune_recurrent_fp32io16_forward(sco, cs, ce, state, *toks, y, boundary, sda, g["scale"])
    torch.cuda.synchronize()
    for got, name in zip((y, state, boundary, sda), ("y", "final_state", "boundary", "state_dot_a")):
        assert torch.allclose(got.float().cpu(), g[name].float(), atol=3e-4, rtol=3e-4), name
    # the golden loss is sum(y^2) + sum(final^2)
    go = (2 * y.float()).to(y.dtype)
    gf = 2 * state
    grads = [torch.empty_like(t) for t in toks] + [torch.empty_like(state)]
    C.statetune_recurrent_fp32io16_backward(sco, cs, ce, state, *toks, sda, go, gf, boundary, *grads[:3], None,
                                            *grads[4:], g["scale"])
    torch.cuda.synchronize()
    for t, name in zip(grads, ("dr", "dw", "dk", "dv", "da", "db", "dS0")):
        if name == "dv":
            continue  # passed as None: not wanted
        assert torch.allclose(t.float().cpu(), g[name], atol=6e-4, rtol=6e-3), name


def test_dense_op_library_checkpoints_and_gradients(oracle):
    """torch.ops.rwkv7_clampw_v3 at T = 208 (three full 64-token chunks and a 16-token tail): `s` holds the oracle's
    state after every 16 tokens, `sa` its state_dot_a rows, and the backward (which takes every fourth checkpoint
    as a chunk boundary) gives the gradients of the oracle's float64 backward."""
    import flashrwkv_b200
    from flashrwkv_b200._ext import extension

    native = extension()  # loading the native module registers the op library
    B, T, H = 2, 208, 2
    gen = torch.Generator().manual_seed(20260806)
    four = [(torch.randn(B, T, H, 64, generator=gen) * sc).to(torch.bfloat16).cuda()
            for sc in (0.12, 2.0, 0.1, 0.1, 0.1, 0.1)]
    dy = (torch.randn(B, T, H, 64, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    y = torch.empty_like(four[3])
    s = torch.full((B, H, T // 16, 64, 64), float("nan"), device="cuda")
    sa = torch.full((B, T, H, 64), float("nan"), device="cuda")
    torch.ops.rwkv7_clampw_v3.forward(*four, y, s, sa, 64)
    grads = [torch.full_like(four[0], float("nan")) for _ in range(6)]
    torch.ops.rwkv7_clampw_v3.backward(*four, dy, s, sa, *grads, 64)
    torch.cuda.synchronize()
    G = T // 16
    cs = torch.arange(G, dtype=torch.int32) * 16
    cu = torch.tensor([0, T], dtype=torch.int32)
    for bi in range(B):
        packed = [t[bi].float().cpu() for t in four]
        want = oracle.forward(*packed, state_pool=torch.zeros(1, H, 64, 64), cu_seqlens=cu,
                              chunks=(torch.tensor([0, G], dtype=torch.int32), cs, cs + 16), want_state_dot_a=True)
        assert rel_rmse(y[bi].float().cpu(), want["y"]) <= 8e-3
        assert rel_rmse(sa[bi].cpu(), want["state_dot_a"]) <= 3e-3
        for c in range(G):
            after = want["boundary"][c + 1] if c + 1 < G else want["state_pool"][0]
            assert rel_rmse(s[bi, :, c].cpu(), after) <= 3e-3, (bi, c)
            assert max_abs(s[bi, :, c].cpu(), after) <= 3e-3 * float(abs(after).max()) + 1e-5, (bi, c)
        back = oracle.backward(*packed, initial_state=torch.zeros(1, H, 64, 64), cu_seqlens=cu,
                               grad_output=dy[bi].float().cpu())
        for got, name in zip(grads, ("r", "decay_logits", "k", "v", "a", "b")):
            assert torch.isfinite(got).all()
            assert rel_rmse(got[bi].float().cpu(), back[name]) <= 1.5e-2, name
    assert all(int(f.item()) == 0 for f in native.rwkv7_clampw_v3_error_flags())


@pytest.mark.parametrize("head_size", [128, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_wide_head_statetune_vs_oracle(oracle, head_size, dtype):
    """Head sizes 128 and 256: outputs, saved tensors and all seven gradients against the oracle's float64 forward
    and backward; ragged chunks (a 16-token multiple, a tail of 1, chunks that need one, two and three checkpoints),
    non-zero initial state, upstream gradients on the output and on the final state."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata

    lengths = (81, 1, 48)
    H, D, B, N = 2, head_size, len(lengths), sum(lengths)
    toks = [t.to(dtype) for t in synthetic.wkv7_inputs(N, H, D, seed=41 + D, dtype=torch.float32)]
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    S0 = synthetic.state_pool(B, H, D, seed=6)
    gen = torch.Generator().manual_seed(9)
    dy = torch.randn(N, H, D, generator=gen).to(dtype)
    dSf = torch.randn(B, H, D, D, generator=gen) * 0.1
    meta = make_chunk_metadata(cu.cuda(), 64)
    fwd = oracle.forward(*toks, state_pool=S0, cu_seqlens=cu, scale=0.8, chunks=tuple(m.cpu() for m in meta),
                         want_state_dot_a=True)
    want = oracle.backward(*toks, initial_state=S0, cu_seqlens=cu, grad_output=dy, grad_final_state=dSf, scale=0.8)
    dS0 = S0.cuda().requires_grad_()
    dtoks = [t.cuda().requires_grad_() for t in toks]
    out = F.statetune_recurrent_fp32io16(dS0, *meta, *dtoks, scale=0.8)
    tol = 8e-3 if dtype == torch.bfloat16 else 2e-3
    assert rel_rmse(out[0].detach().float().cpu(), fwd["y"]) <= tol
    assert rel_rmse(out[1].detach().cpu(), fwd["state_pool"]) <= 1e-4
    assert rel_rmse(out[2].detach().cpu(), fwd["boundary"]) <= 1e-4
    assert rel_rmse(out[3].detach().cpu(), fwd["state_dot_a"]) <= 1e-4
    torch.autograd.backward([out[0], out[1]], [dy.cuda(), dSf.cuda()])
    for t, name in zip(dtoks, ("r", "decay_logits", "k", "v", "a", "b")):
        assert torch.isfinite(t.grad).all()
        assert rel_rmse(t.grad.float().cpu(), want[name]) <= tol, name
    assert rel_rmse(dS0.grad.cpu(), want["initial_state"]) <= 1e-3
    # bit-identical on a second run (fixed-order sums over the column blocks)
    dtoks2 = [t.detach().clone().requires_grad_() for t in dtoks]
    dS02 = S0.cuda().requires_grad_()
    out2 = F.statetune_recurrent_fp32io16(dS02, *meta, *dtoks2, scale=0.8)
    torch.autograd.backward([out2[0], out2[1]], [dy.cuda(), dSf.cuda()])
    for t, t2 in zip(dtoks, dtoks2):
        assert torch.equal(t.grad, t2.grad)


@pytest.mark.parametrize("head_size", [128, 256])
def test_wide_head_pretrain_and_op_library(oracle, head_size):
    """The dense pretraining operator at head sizes 128 / 256 through this package's wrapper and through
    torch.ops.rwkv7_clampw_v3 (16-token checkpoints, sa, gradients written into the caller's tensors)."""
    import flashrwkv_b200 as F

    B, T, H, D = 2, 80, 1, head_size
    gen = torch.Generator().manual_seed(20260806 + D)
    vals = [(torch.randn(B, T, H * D, generator=gen) * sc).to(torch.bfloat16).cuda().requires_grad_()
            for sc in (0.12, 2.0, 0.1, 0.1, 0.1, 0.1)]
    dy = (torch.randn(B, T, H * D, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    y = F.pretrain_recurrent_bf16(*vals, head_size=D)
    y.backward(dy)
    four = [v.detach().view(B, T, H, D) for v in vals]
    out = torch.empty_like(four[3])
    s = torch.full((B, H, T // 16, D, D), float("nan"), device="cuda")
    sa = torch.full((B, T, H, D), float("nan"), device="cuda")
    torch.ops.rwkv7_clampw_v3.forward(*four, out, s, sa, D)
    grads = [torch.full_like(four[0], float("nan")) for _ in range(6)]
    torch.ops.rwkv7_clampw_v3.backward(*four, dy.view(B, T, H, D), s, sa, *grads, D)
    assert torch.equal(out.view(B, T, H * D), y.detach())
    G = T // 16
    cs = torch.arange(G, dtype=torch.int32) * 16
    cu = torch.tensor([0, T], dtype=torch.int32)
    for bi in range(B):
        packed = [t[bi].float().cpu() for t in four]
        want = oracle.forward(*packed, state_pool=torch.zeros(1, H, D, D), cu_seqlens=cu,
                              chunks=(torch.tensor([0, G], dtype=torch.int32), cs, cs + 16), want_state_dot_a=True)
        assert rel_rmse(out[bi].float().cpu(), want["y"]) <= 8e-3
        assert rel_rmse(sa[bi].cpu(), want["state_dot_a"]) <= 1e-4
        for c in range(G):
            after = want["boundary"][c + 1] if c + 1 < G else want["state_pool"][0]
            assert rel_rmse(s[bi, :, c].cpu(), after) <= 1e-4, (bi, c)
        back = oracle.backward(*packed, initial_state=torch.zeros(1, H, D, D), cu_seqlens=cu,
                               grad_output=dy.view(B, T, H, D)[bi].float().cpu())
        for got, v, name in zip(grads, vals, ("r", "decay_logits", "k", "v", "a", "b")):
            assert rel_rmse(got[bi].float().cpu(), back[name]) <= 8e-3, name
            assert torch.equal(got.view(B, T, H * D), v.grad), name


def test_chunk_tables_are_validated_before_any_launch():
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    H, D, N = 1, 64, 40
    toks = [t.cuda() for t in synthetic.wkv7_inputs(N, H, D, seed=3)]
    S0 = torch.zeros(2, H, D, D, device="cuda")
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    good = (i32([0, 1, 2]), i32([0, 30]), i32([30, 40]))
    F.statetune_recurrent_fp32io16(S0, *good, *toks)
    bad = {
        "0 <= start <= end <= total_tokens": (i32([0, 1, 2]), i32([0, 30]), i32([30, 41])),
        "0 <= start <= end": (i32([0, 1, 2]), i32([5, 30]), i32([3, 40])),
        "rise from 0": (i32([0, 2, 1]), i32([0, 30]), i32([30, 40])),
        "number of chunks": (i32([0, 1, 3]), i32([0, 30]), i32([30, 40])),
        "contiguous": (i32([0, 2, 2]), i32([0, 31]), i32([30, 40])),
    }
    for match, tables in bad.items():
        with pytest.raises(ValueError, match=match):
            F.statetune_recurrent_fp32io16(S0, *tables, *toks)


def test_device_error_words_are_kept_and_zero_after_clean_runs():
    """Every stage with bounded waits leaves its error word where `device_error_flags()` finds it; clean runs read 0
    and `check_device_error_flags()` stays silent.  (The give-up path itself is exercised on a barrier at which
    nothing arrives: tests/test_umma_gpu.py, and by the sticky time-out bit of the decode operators.)"""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata

    H, D, T = 2, 64, 130
    toks = [t.cuda().requires_grad_() for t in synthetic.wkv7_inputs(T, H, D, seed=2)]
    S0 = synthetic.state_pool(1, H, D, seed=3, device="cuda").requires_grad_()
    cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    out = F.statetune_recurrent_fp32io16(S0, *make_chunk_metadata(cu, 64), *toks)
    out[0].float().sum().backward()
    x = torch.randn(40, 256, device="cuda").to(torch.bfloat16)
    W = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    F.infer_tmix_linear_forward_varlen(x, W)  # more than 8 rows: the tensor-core GEMM
    flags = F.device_error_flags()
    for stage in ("wkv7_chunk_forward", "wkv7_chunk_backward", "tmix_linear"):
        assert flags.get(stage) == 0, (stage, flags)
    F.check_device_error_flags()


def test_chunks_longer_than_64_tokens_are_split_internally(oracle):
    """Caller-built tables with chunks of 100 and 150 tokens (the reference accepts any chunk length): outputs,
    boundaries named by the caller's table and all seven gradients against the oracle."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    H, D = 2, 64
    lengths = (250, 70)
    N = sum(lengths)
    toks = synthetic.wkv7_inputs(N, H, D, seed=77)
    S0 = synthetic.state_pool(2, H, D, seed=78)
    sco = torch.tensor([0, 2, 3], dtype=torch.int32)
    cs = torch.tensor([0, 100, 250], dtype=torch.int32)
    ce = torch.tensor([100, 250, 320], dtype=torch.int32)
    cu = torch.tensor([0, 250, 320], dtype=torch.int32)
    gen = torch.Generator().manual_seed(5)
    dy = torch.randn(N, H, D, generator=gen).to(torch.bfloat16)
    fwd = oracle.forward(*toks, state_pool=S0, cu_seqlens=cu, chunks=(sco, cs, ce), want_state_dot_a=True)
    want = oracle.backward(*toks, initial_state=S0, cu_seqlens=cu, grad_output=dy)
    dS0 = S0.cuda().requires_grad_()
    dtoks = [t.cuda().requires_grad_() for t in toks]
    out = F.statetune_recurrent_fp32io16(dS0, sco.cuda(), cs.cuda(), ce.cuda(), *dtoks)
    assert out[2].shape == (3, H, D, D)
    assert rel_rmse(out[0].detach().float().cpu(), fwd["y"]) <= 8e-3
    assert rel_rmse(out[1].detach().cpu(), fwd["state_pool"]) <= 1e-3
    assert rel_rmse(out[2].detach().cpu(), fwd["boundary"]) <= 1e-3
    assert rel_rmse(out[3].detach().cpu(), fwd["state_dot_a"]) <= 3e-3
    out[0].backward(dy.cuda())
    for t, name in zip(dtoks, ("r", "decay_logits", "k", "v", "a", "b")):
        assert rel_rmse(t.grad.float().cpu(), want[name]) <= 8e-3, name
    assert rel_rmse(dS0.grad.cpu(), want["initial_state"]) <= 8e-3


@pytest.mark.parametrize("head_size", [64, 128])
def test_native_training_entries_fail_closed_on_bad_chunk_tables(head_size):
    """The reference-named native entries are reached with caller-built tables (the reference's wrapper checks shapes
    only).  A table with a chunk of 70 tokens, or one that ends beyond the token count, gets its verdict on the device:
    outputs and gradients read as NaN, the state keeps its value, nothing is accessed out of range, no host sync."""
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200._ext import extension

    C_ = extension()
    H, D, N = 1, head_size, 100
    toks = [t.cuda() for t in synthetic.wkv7_inputs(N, H, D, seed=5)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    for cs, ce in (([0, 70], [70, 100]), ([0, 50], [50, 164])):
        sco = i32([0, 2])
        state = synthetic.state_pool(1, H, D, seed=6, device="cuda")
        before = state.clone()
        out = torch.zeros_like(toks[3])
        boundary = torch.zeros(2, H, D, D, device="cuda")
        sda = torch.zeros(N, H, D, device="cuda")
        C_.statetune_recurrent_fp32io16_forward(sco, i32(cs), i32(ce), state, *toks, out, boundary, sda, 1.0)
        torch.cuda.synchronize()
        assert torch.isnan(out.float()).all()
        assert torch.equal(state, before)
        grads = [torch.zeros_like(toks[0]) for _ in range(6)]
        dS0 = torch.zeros_like(state)
        C_.statetune_recurrent_fp32io16_backward(sco, i32(cs), i32(ce), state, *toks, sda, torch.ones_like(toks[0]), None,
                                                 boundary, *grads, dS0, 1.0)
        torch.cuda.synchronize()
        for g in grads:
            assert torch.isnan(g.float()).all()


def test_c_abi_chunked_backward_with_decay_bias_vs_oracle(oracle):
    """The three native stages (fused forward with saved tensors, adjoint scan, chunk-parallel backward) called with
    raw pointers and a per-head decay bias, which the Python training operators never pass: the adjoint scan makes its
    keys from the decay tile, so the bias must reach them through it.  All seven gradients against the oracle."""
    import ctypes

    from flashrwkv_b200 import _ext, synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata, wkv7_chunk_forward

    lib = _ext.capi()
    lengths = (130, 64, 200)
    H, D, B, N = 2, 64, len(lengths), sum(lengths)
    toks = synthetic.wkv7_inputs(N, H, D, seed=77)
    gen = torch.Generator().manual_seed(9)
    bias = (torch.randn(H, D, generator=gen) * 0.5).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32)
    S0 = synthetic.state_pool(B, H, D, seed=6)
    dy = torch.randn(N, H, D, generator=gen).to(torch.bfloat16)
    dSf = torch.randn(B, H, D, D, generator=gen) * 0.1
    want = oracle.backward(*toks, initial_state=S0, cu_seqlens=cu, grad_output=dy, grad_final_state=dSf, scale=0.9,
                           decay_bias=bias)
    dt = [t.cuda() for t in toks]
    sco, cs, ce = make_chunk_metadata(cu.cuda(), 64)
    state = S0.cuda().clone()
    sda = torch.empty(N, H, D, device="cuda")
    _, boundary, flag = wkv7_chunk_forward(*dt, state=state, chunk_metadata=(sco, cs, ce), scale=0.9,
                                           decay_bias=bias.cuda(), want_boundary=True, state_dot_a=sda, path=1)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    r, w, k, v, a, b = dt
    bias_d, dy_d = bias.cuda(), dy.cuda()
    g_state = dSf.cuda().clone()
    adjoint = torch.empty(cs.numel(), H, D, D, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.frwkv_wkv7_adjoint_scan(p(sco), p(cs), p(ce), p(r), p(w), p(a), p(b), p(bias_d), p(dy_d), p(g_state),
                                     p(adjoint), p(err), None, N, B, cs.numel(), H, D, 1, ctypes.c_float(0.9), stream)
    assert rc == 0, lib.frwkv_last_error()
    grads = [torch.empty_like(r) for _ in range(6)]  # dr, dw, dk, dv, da, db
    rc = lib.frwkv_wkv7_chunk_backward(p(sco), p(cs), p(ce), p(state), p(boundary), p(adjoint), p(sda), p(r), p(w),
                                       p(k), p(v), p(a), p(b), p(bias_d), p(dy_d), *(p(t) for t in grads), p(err), None,
                                       N, B, cs.numel(), H, D, 1, ctypes.c_float(0.9), stream)
    assert rc == 0, lib.frwkv_last_error()
    torch.cuda.synchronize()
    assert int(flag.item()) == 0 and int(err.item()) == 0
    for got, name in zip(grads, ("r", "decay_logits", "k", "v", "a", "b")):
        assert rel_rmse(got.float().cpu(), want[name]) <= 8e-3, name
    assert rel_rmse(g_state.cpu(), want["initial_state"]) <= 8e-3
