"""Parity of the TMix kernels (token shift, per-head ops, projections) with the CPU oracle and the golden vectors.

Tolerances: elementwise / per-head outputs must be the oracle's value up to one rounding of the 16-bit output
(relative RMSE <= 1.5e-3 fp16, 4e-3 bf16); projections the same (fp32 accumulation over K <= 2048); the
reference's own allclose(atol=rtol=0.04) bounds (tests/tmix/*/test.py) are far looser and implied.
"""
import numpy as np
import pytest
import torch

from _util import load_golden, max_abs, rel_rmse

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 1.5e-3, torch.bfloat16: 4e-3}


def _c(*ts):
    return [t.cuda() for t in ts]


def test_golden_mix6_ticket_and_shift_update():
    import flashrwkv_b200 as F

    g = load_golden("tmix_mix6")
    x, pool = g["x"].cuda(), g["shift_pool"].cuda().clone()
    cu, idx = g["cu_seqlens"].cuda(), g["state_indices"].cuda()
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=5, state_pool_size=4)
    outs = F.infer_tmix_mix6_forward_varlen(x, *g["mix"].cuda().unbind(0), shift_state_pool=pool, cu_seqlens=cu,
                                            state_indices=idx, validated_metadata=ticket)
    torch.cuda.synchronize()
    for j in range(6):
        assert torch.allclose(outs[j].float().cpu(), g["out"][j], atol=0.01, rtol=0.01)
    assert torch.equal(pool.cpu(), g["shift_after"])
    cu[1] += 1
    before = pool.clone()
    with pytest.raises(RuntimeError, match="version"):
        F.infer_tmix_mix6_forward_varlen(x, *g["mix"].cuda().unbind(0), shift_state_pool=pool, cu_seqlens=cu,
                                         state_indices=idx, validated_metadata=ticket)
    assert torch.equal(pool, before)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("lengths", [(1,) * 7, (3, 1, 64, 2)])
def test_mix6_vs_oracle(oracle, dtype, lengths):
    import flashrwkv_b200 as F

    C, N = 2048, sum(lengths)
    gen = torch.Generator().manual_seed(N)
    x = torch.randn(N, C, generator=gen).to(dtype)
    mixes = [torch.rand(C, generator=gen).to(dtype) for _ in range(6)]
    pool = torch.randn(len(lengths) + 3, C, generator=gen).to(dtype)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
    idx = torch.randperm(len(lengths) + 3, generator=gen)[: len(lengths)].to(torch.int32)
    want, want_pool = oracle.mix6(x, pool, mixes, cu, idx)
    dpool = pool.cuda()
    outs = F.infer_tmix_mix6_forward_varlen(x.cuda(), *_c(*mixes), shift_state_pool=dpool, cu_seqlens=cu.cuda(),
                                            state_indices=idx.cuda(),
                                            max_seqlen=max(lengths))
    torch.cuda.synchronize()
    for j in range(6):
        assert rel_rmse(outs[j].float().cpu(), want[j]) <= TOL[dtype]
    assert torch.equal(dpool.float().cpu(), torch.from_numpy(want_pool))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("head_size", [64, 128, 256])
def test_per_head_ops_vs_oracle(oracle, dtype, head_size):
    import flashrwkv_b200 as F

    N, C = 37, 2048
    gen = torch.Generator().manual_seed(4)
    rn = lambda *s: torch.randn(*s, generator=gen).to(dtype)  # noqa: E731
    k, a12, k_k, a0, k_a = rn(N, C), rn(N, C), rn(C), rn(C), rn(C)
    got = F.infer_tmix_kk_a_gate_forward_varlen(*_c(k, k_k, a0, a12, k_a), head_size=head_size)
    for o, w in zip(got, oracle.kk_a_gate(k, k_k, a0, a12, k_a, head_size=head_size)):
        assert rel_rmse(o.float().cpu(), w) <= TOL[dtype]
    x, r, kk, v, g, r_k, wt, bs = rn(N, C), rn(N, C), rn(N, C), rn(N, C), rn(N, C), rn(C), rn(C), rn(C)
    got = F.infer_tmix_lnx_rkvres_xg_forward_varlen(*_c(x, r, kk, v, r_k, wt, bs, g), head_size=head_size)
    assert rel_rmse(got.float().cpu(), oracle.lnx_rkvres_xg(x, r, kk, v, r_k, wt, bs, g, head_size=head_size)) <= TOL[dtype]
    v, vf, v12, v0 = rn(N, C), rn(N, C), rn(N, C), rn(C)
    got = F.infer_tmix_vres_gate_forward_varlen(*_c(v, vf, v0, v12))
    assert rel_rmse(got.float().cpu(), oracle.vres_gate(v, vf, v0, v12)) <= TOL[dtype]


def test_golden_per_head_and_known_answers():
    import flashrwkv_b200 as F

    g = load_golden("tmix_kk_a_gate")
    outs = F.infer_tmix_kk_a_gate_forward_varlen(*_c(g["k"], g["k_k"], g["a0"], g["a12"], g["k_a"]))
    for o, name in zip(outs, ("new_k", "neg_kk", "kka")):
        assert torch.allclose(o.float().cpu(), g[name], atol=0.04, rtol=0.04)
        assert rel_rmse(o.float().cpu(), g[name]) <= TOL[torch.float16]
    g = load_golden("tmix_lnx")
    out = F.infer_tmix_lnx_rkvres_xg_forward_varlen(*_c(g["x"], g["r"], g["k"], g["v"], g["r_k"], g["weight"],
                                                       g["bias"], g["g"]))
    assert rel_rmse(out.float().cpu(), g["out"]) <= TOL[torch.float16]
    g = load_golden("tmix_vres")
    out = F.infer_tmix_vres_gate_forward_varlen(*_c(g["v"], g["v_first"], g["v0"], g["v12"]))
    assert rel_rmse(out.float().cpu(), g["out"]) <= TOL[torch.float16]
    ones = torch.ones(65536, 4096, dtype=torch.float16, device="cuda")
    vec = torch.ones(4096, dtype=torch.float16, device="cuda")
    new_k, neg_kk, kka = F.infer_tmix_kk_a_gate_forward_varlen(ones, vec, 0 * vec, 0 * ones, vec)
    for o, val in ((new_k, 0.5), (neg_kk, -0.125), (kka, 0.0625)):
        assert torch.allclose(o[[0, -1]].float(), torch.full_like(o[[0, -1]].float(), val))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 4, 5, 7, 8, 9, 130, 512])
def test_lowrank_group_and_dense_linear_vs_oracle(oracle, dtype, M):
    import flashrwkv_b200 as F

    C, ranks = 2048, {"w": 96, "a": 96, "g": 256, "v": 64}
    gen = torch.Generator().manual_seed(100 + M)
    rn = lambda *s, scale=1.0: (torch.randn(*s, generator=gen) * scale).to(dtype)  # noqa: E731
    xs = {n: rn(M, C) for n in "wagv"}
    w1 = {n: rn(ranks[n], C, scale=0.02) for n in "wagv"}
    w2 = {n: rn(C, ranks[n], scale=0.02) for n in "wagv"}
    tol = TOL[dtype]
    rank_feats = F.infer_tmix_lowrank_wagv_in_forward_varlen(*_c(*(xs[n] for n in "wagv")), *_c(*(w1[n] for n in "wagv")))
    feats = {}
    for n, got in zip("wagv", rank_feats):
        assert got.shape == (M, ranks[n])
        assert rel_rmse(got.float().cpu(), oracle.linear_nt(xs[n], w1[n])) <= tol
        feats[n] = got.cpu()
    three = F.infer_tmix_lowrank_in_forward_varlen(*_c(xs["w"], xs["a"], xs["g"]), *_c(w1["w"], w1["a"], w1["g"]))
    for n, got in zip("wag", three):
        assert torch.equal(got.cpu(), feats[n])
    v, v_first, v0 = rn(M, C), rn(M, C), rn(C)
    outs = F.infer_tmix_lowrank_vres_forward_varlen(*_c(*(feats[n] for n in "wagv")), *_c(*(w2[n] for n in "wagv")),
                                                    *_c(v, v_first, v0))
    acts = {"w": "tanh", "a": "none", "g": "sigmoid"}
    for n, got in zip("wag", outs[:3]):
        assert rel_rmse(got.float().cpu(), oracle.linear_nt(feats[n], w2[n], act=acts[n])) <= 2 * tol
    v12 = oracle.linear_nt(feats["v"], w2["v"])
    assert rel_rmse(outs[3].float().cpu(), oracle.vres_gate(v, v_first, v0, v12)) <= 2 * tol
    plain = F.infer_tmix_lowrank_out_forward_varlen(*_c(*(feats[n] for n in "wag")), *_c(*(w2[n] for n in "wag")))
    for got, ref in zip(plain, outs[:3]):
        assert torch.equal(got, ref)
    W = rn(C, C, scale=0.02)
    y = F.infer_tmix_linear_forward_varlen(xs["w"].cuda(), W.cuda())
    assert rel_rmse(y.float().cpu(), oracle.linear_nt(xs["w"], W)) <= tol
    with pytest.raises(ValueError, match="R <= 512"):
        F.infer_tmix_linear_rank_in_forward_varlen(xs["w"].cuda(), weight_t=rn(520, C).cuda())
    with pytest.raises(ValueError, match="runtime layout"):
        F.infer_tmix_linear_rank_in_forward_varlen(xs["w"].cuda(), weight=rn(C + 8, 96).cuda())
    # the same projections from weights held only in the runtime layout [K,N]
    kn = {n: w1[n].t().contiguous().cuda() for n in "wagv"}
    rt = F.infer_tmix_lowrank_wagv_in_forward_varlen(*_c(*(xs[n] for n in "wagv")), None, None, None, None,
                                                     **{f"{n}1_runtime": kn[n] for n in "wagv"})
    for n, got in zip("wagv", rt):
        assert rel_rmse(got.float().cpu(), oracle.linear_nt(xs[n], w1[n])) <= tol
    kn2 = {n: w2[n].t().contiguous().cuda() for n in "wagv"}
    rt2 = F.infer_tmix_lowrank_vres_forward_varlen(*_c(*(feats[n] for n in "wagv")), None, None, None, None,
                                                   *_c(v, v_first, v0), **{f"{n}2_runtime": kn2[n] for n in "wagv"})
    for got, ref in zip(rt2, outs):
        assert rel_rmse(got.float().cpu(), ref.float().cpu()) <= tol
    one = F.infer_tmix_linear_rank_out_tanh_forward_varlen(feats["w"].cuda(), weight=kn2["w"])
    assert rel_rmse(one.float().cpu(), outs[0].float().cpu()) <= tol


def test_golden_lowrank_pair():
    import flashrwkv_b200 as F

    g = load_golden("tmix_lowrank")
    rank = F.infer_tmix_linear_rank_in_forward_varlen(g["x"].cuda(), weight_t=g["w1"].cuda())
    assert torch.allclose(rank.float().cpu(), g["rank"].float(), atol=0.04, rtol=0.04)
    assert rel_rmse(rank.float().cpu(), g["rank"].float()) <= TOL[torch.float16]
    out = F.infer_tmix_linear_rank_out_tanh_forward_varlen(g["rank"].cuda(), weight_t=g["w2"].cuda())
    assert rel_rmse(out.float().cpu(), g["out_tanh"]) <= TOL[torch.float16]


def test_elementwise_activations():
    import flashrwkv_b200 as F

    x = torch.randn(37, 96, generator=torch.Generator().manual_seed(1)).half()
    assert rel_rmse(F.infer_tmix_linear_act_tanh_forward_varlen(x.cuda()).float().cpu(), torch.tanh(x.float())) <= 1e-3
    assert rel_rmse(F.infer_tmix_linear_act_sigmoid_forward_varlen(x.cuda()).float().cpu(),
                    torch.sigmoid(x.float())) <= 1e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(300, 72, 200), (129, 264, 2048), (4096, 2048, 2048), (1000, 520, 72)])
def test_dense_linear_ragged_shapes(oracle, dtype, shape):
    """Row, column and K counts that are not multiples of the tensor-core tile, and a many-tile case."""
    import flashrwkv_b200 as F

    M, N, K = shape
    gen = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=gen).to(dtype)
    W = (torch.randn(N, K, generator=gen) * 0.05).to(dtype)
    y = F.infer_tmix_linear_forward_varlen(x.cuda(), W.cuda())
    ref = x.double() @ W.double().T
    assert y.shape == (M, N)
    assert rel_rmse(y.double().cpu(), ref) <= TOL[dtype]
    assert max_abs(y.double().cpu(), ref) <= 8 * TOL[dtype] * float(ref.abs().max())
    if N % 8 == 0:  # the runtime layout [K,N] read in place (rows of N must be 16-byte aligned)
        y_kn = F.infer_tmix_linear_forward_varlen(x.cuda(), W.t().contiguous().cuda(), weight_is_transposed=True)
        assert y_kn.shape == (M, N)
        assert rel_rmse(y_kn.double().cpu(), ref) <= TOL[dtype]
        assert max_abs(y_kn.double().cpu(), ref) <= 8 * TOL[dtype] * float(ref.abs().max())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("lengths", [(1,), (1,) * 7, (3, 1, 2), (8,), (5, 30), (1,) * 130, (127, 1, 2, 129, 64, 200),
                                     (300,)])
@pytest.mark.parametrize("C", [512, 328])
def test_shift_project_fused_vs_oracle(oracle, dtype, lengths, C):
    """Token shift fused into the projections (<= 8 rows: the small-row kernel; more rows with fuse_many_rows: inside
    the TMA-fed tensor-core GEMM, on its staged x tiles) against mix6 and the projection of the oracle; sequence starts inside,
    at the first and at the last row of a 128-row tile, rows and channels that do not fill a tile (C = 328 leaves a
    partial k-block); the shift states end up holding each sequence's last row."""
    import flashrwkv_b200 as F

    M, slots = sum(lengths), len(lengths) + 3
    gen = torch.Generator().manual_seed(31 * M + len(lengths))
    x = torch.randn(M, C, generator=gen).to(dtype)
    pool = torch.randn(slots, C, generator=gen).to(dtype)
    mix = [torch.rand(C, generator=gen).to(dtype) for _ in range(4)]
    Ws = [(torch.randn(n, C, generator=gen) * 0.05).to(dtype) for n in (512, 96, 64, 256, 512)]
    use = [0, 1, 2, 3, 2]  # the fifth projection shares the third mix vector
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
    idx = torch.randperm(slots, generator=gen)[:len(lengths)].int()
    d_pool = pool.cuda().clone()
    outs = F.infer_tmix_shift_project_forward_varlen(x.cuda(), [mix[u].cuda() for u in use], [w.cuda() for w in Ws],
                                                     shift_state_pool=d_pool, cu_seqlens=cu.cuda(),
                                                     state_indices=idx.cuda(), fuse_many_rows=True)
    torch.cuda.synchronize()
    # reference: previous rows, fp32 interpolation, projection
    prev = torch.empty(M, C)
    for s, (a, b) in enumerate(zip(cu[:-1].tolist(), cu[1:].tolist())):
        prev[a] = pool[idx[s]].float()
        prev[a + 1:b] = x[a:b - 1].float()
    for j, (u, w) in enumerate(zip(use, Ws)):
        mixed = x.float() + (prev - x.float()) * mix[u].float()
        ref = mixed.double() @ w.double().T
        assert outs[j].shape == (M, w.shape[0])
        assert rel_rmse(outs[j].double().cpu(), ref) <= 2 * TOL[dtype], f"projection {j}"
    expect_pool = pool.clone()
    for s, b in enumerate(cu[1:].tolist()):
        expect_pool[idx[s]] = x[b - 1]
    assert torch.equal(d_pool.cpu(), expect_pool)
    if M > 8:  # the default for many rows (mix6, then the GEMMs) rounds the interpolated rows to 16 bits in between
        d_pool3 = pool.cuda().clone()
        outs3 = F.infer_tmix_shift_project_forward_varlen(x.cuda(), [mix[u].cuda() for u in use], [w.cuda() for w in Ws],
                                                          shift_state_pool=d_pool3, cu_seqlens=cu.cuda(),
                                                          state_indices=idx.cuda())
        for a, b in zip(outs, outs3):
            assert rel_rmse(a.double().cpu(), b.double().cpu()) <= 2 * TOL[dtype]
        assert torch.equal(d_pool3.cpu(), expect_pool)
    if M > 8 and len(lengths) > 1:  # bad metadata (a slot used twice) fails closed: NaN outputs, shift states untouched
        bad = idx.clone()
        bad[-1] = bad[0]
        d_pool2 = pool.cuda().clone()
        outs2 = F.infer_tmix_shift_project_forward_varlen(x.cuda(), [mix[u].cuda() for u in use], [w.cuda() for w in Ws],
                                                          shift_state_pool=d_pool2, cu_seqlens=cu.cuda(),
                                                          state_indices=bad.cuda(), fuse_many_rows=True)
        torch.cuda.synchronize()
        assert all(bool(torch.isnan(o.float()).all()) for o in outs2)
        assert torch.equal(d_pool2.cpu(), pool)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_add_layer_norm_family(oracle, dtype):
    """add, LayerNorm, add + LayerNorm (both outputs / last only) against the oracle; the sum is the exactly rounded
    16-bit sum (reference: tests/tmix/normalization/test.py:17-88)."""
    import flashrwkv_b200 as F

    gen = torch.Generator().manual_seed(54)
    for rows, C in ((5, 8), (4, 4096), (193, 2048)):
        x = torch.randn(rows, C, generator=gen).to(dtype)
        res = torch.randn(rows, C, generator=gen).to(dtype)
        w = torch.randn(C, generator=gen).to(dtype)
        b = torch.randn(C, generator=gen).to(dtype)
        dx, dr, dw, db = x.cuda(), res.cuda(), w.cuda(), b.cuda()
        exact_sum = (x.float() + res.float()).to(dtype)
        assert torch.equal(F.infer_tmix_add_forward_varlen(dx, dr).cpu(), exact_sum)
        ln = F.infer_tmix_layer_norm_forward_varlen(dx, dw, db)
        assert rel_rmse(ln.float().cpu(), oracle.layer_norm(x, w, b)) <= TOL[dtype]
        s, n = F.infer_tmix_add_layer_norm_forward_varlen(dx, dr, dw, db, batch_size=min(2, rows))
        ref_sum, ref_norm = oracle.layer_norm(x, w, b, residual=res, io_dtype=dtype)
        assert torch.equal(s.cpu(), exact_sum)
        assert rel_rmse(n.float().cpu(), ref_norm) <= TOL[dtype]
        last = F.infer_tmix_add_last_layer_norm_forward_varlen(dx, dr, dw, db, eps=1e-5)
        assert torch.equal(last, n)
    with pytest.raises(ValueError, match="eps"):
        F.infer_tmix_layer_norm_forward_varlen(dx, dw, db, eps=0.0)
    with pytest.raises(ValueError, match="same shape"):
        F.infer_tmix_add_forward_varlen(dx, dr[:-1])


def test_golden_mix6_add_layer_norm_fused_and_composed():
    """The fused one-kernel form (one-token sequences) and the composed form give the golden outputs of the
    reference's formulas, and the shift states receive the normalised rows."""
    import flashrwkv_b200 as F

    g = load_golden("tmix_norm")
    mix = [m.cuda() for m in g["mix"]]
    for max_seqlen in (1, None):
        pool = g["shift_pool"].cuda().clone()
        outs = F.infer_tmix_mix6_add_layer_norm_forward_varlen(
            g["x"].cuda(), g["residual"].cuda(), g["weight"].cuda(), g["bias"].cuda(), *mix, shift_state_pool=pool,
            cu_seqlens=g["cu_seqlens"].cuda(), state_indices=g["state_indices"].cuda(), max_seqlen=max_seqlen)
        torch.cuda.synchronize()
        assert len(outs) == 7
        assert torch.equal(outs[0].cpu(), g["sum"])
        for j in range(6):
            assert torch.allclose(outs[1 + j].float().cpu(), g["mixed"][j], atol=0.01, rtol=0.01)
            assert rel_rmse(outs[1 + j].float().cpu(), g["mixed"][j]) <= TOL[torch.float16]
        assert torch.allclose(pool.float().cpu(), g["shift_after"].float(), atol=0.01, rtol=0.01)
        untouched = [1, 2]
        assert torch.equal(pool[untouched].cpu(), g["shift_pool"][untouched])
