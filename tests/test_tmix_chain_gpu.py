"""The whole RWKV-7 TMix inference layer as one checked chain, through the public operators:

    mix6 -> r/k/v projections + four rank-in products -> rank-out (tanh / sigmoid) + value-residual gate
         -> kk_a_gate -> WKV7 recurrence -> lnx_rkvres_xg -> output projection

at the benchmark's width (C = 2048; ranks 96 / 96 / 64 / 256; head sizes 64, 128, 256), for M in {1, 4, 7, 512} rows
packed as M one-token sequences (decode) and as one M-token sequence (prefill), fp16 and bf16, both with the reference's
operator sequence and with the token shift fused into the projections.  The expected values come from the CPU oracle's
pieces chained the same way, every intermediate rounded to the io type where an operator hands a 16-bit tensor to the
next.  The reference tests the chain as a whole too (tests/tmix/wkv7/test.py:310-414 there, with identity projections);
a transposed mix index or two swapped per-channel vectors passes every single-operator test but not this one.

Bars: relative RMSE of the layer output <= 2.5e-2 (bf16) / 4e-3 (fp16), of the final WKV7 state <= 1e-2 / 2e-3, of
the updated shift state exactly the last row of each sequence.  (One bf16 rounding is 2^-9 = 2e-3 relative; the chain
has about ten of them in sequence, two of them amplified by a 2048-long contraction.)
"""
import numpy as np
import pytest
import torch

from _util import rel_rmse

pytestmark = pytest.mark.gpu

C = 2048
RANKS = {"w": 96, "a": 96, "g": 256, "v": 64}


def _weights(dtype, seed):
    g = torch.Generator().manual_seed(seed)
    wt = lambda n, k: (torch.randn(n, k, generator=g) * 0.02).to(dtype)  # noqa: E731
    vec = lambda lo=0.0, hi=1.0: (torch.rand(C, generator=g) * (hi - lo) + lo).to(dtype)  # noqa: E731
    W = {"Wr": wt(C, C), "Wk": wt(C, C), "Wv": wt(C, C), "Wo": wt(C, C),
         "w1": {n: wt(r, C) for n, r in RANKS.items()}, "w2": {n: wt(C, r) for n, r in RANKS.items()},
         "mix": [vec() for _ in range(6)]}  # mix order: r, w, k, v, a, g
    for name in ("k_k", "a0", "k_a", "r_k", "lnw", "lnb", "v0"):
        W[name] = vec(-0.5, 1.0)
    return W


def _expected(oracle, W, x, v_first, shift0, pool0, cu, idx, D, dtype):
    rd = lambda a: torch.as_tensor(np.asarray(a)).to(dtype).float().numpy()  # noqa: E731  one 16-bit hand-over
    f = lambda t: t.float().numpy()  # noqa: E731
    mixed, shift = oracle.mix6(f(x), f(shift0), [f(m) for m in W["mix"]], cu, idx)
    xr, xw, xk, xv, xa, xg = (rd(m) for m in mixed)
    r = rd(oracle.linear_nt(xr, f(W["Wr"])))
    k = rd(oracle.linear_nt(xk, f(W["Wk"])))
    v = rd(oracle.linear_nt(xv, f(W["Wv"])))
    fw, fa, fg, fv = (rd(oracle.linear_nt(xi, f(W["w1"][n]))) for xi, n in ((xw, "w"), (xa, "a"), (xg, "g"), (xv, "v")))
    w = rd(oracle.linear_nt(fw, f(W["w2"]["w"]), "tanh"))
    a12 = rd(oracle.linear_nt(fa, f(W["w2"]["a"])))
    gate = rd(oracle.linear_nt(fg, f(W["w2"]["g"]), "sigmoid"))
    v12 = oracle.linear_nt(fv, f(W["w2"]["v"]))  # stays fp32 inside the fused value-residual projection
    vres = rd(oracle.vres_gate(v, f(v_first), f(W["v0"]), v12))
    kk, nkk, kka = (rd(t) for t in oracle.kk_a_gate(k, f(W["k_k"]), f(W["a0"]), a12, f(W["k_a"]), D))
    M, H = x.shape[0], C // D
    sh = (M, H, D)
    res = oracle.forward(r.reshape(sh), w.reshape(sh), kk.reshape(sh), vres.reshape(sh), nkk.reshape(sh),
                         kka.reshape(sh), state_pool=pool0, cu_seqlens=cu, state_indices=idx)
    y = rd(res["y"]).reshape(M, C)
    z = rd(oracle.lnx_rkvres_xg(y, r, kk, vres, f(W["r_k"]), f(W["lnw"]), f(W["lnb"]), gate, D))
    out = oracle.linear_nt(z, f(W["Wo"]))
    return out, res["state_pool"], shift


def _layer(F, W, x, v_first, shift, pool, cu, idx, D, fused):
    M, H = x.shape[0], C // D
    lens = (cu[1:] - cu[:-1])
    max_len = int(lens.max().item())
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=M, state_pool_size=pool.shape[0], max_seqlen=max_len)
    w1, w2, mix = W["w1"], W["w2"], W["mix"]
    if fused:
        r, k, v, fw, fa, fg, fv = F.infer_tmix_shift_project_forward_varlen(
            x, [mix[0], mix[2], mix[3], mix[1], mix[4], mix[5], mix[3]],
            [W["Wr"], W["Wk"], W["Wv"], w1["w"], w1["a"], w1["g"], w1["v"]], shift_state_pool=shift, cu_seqlens=cu,
            state_indices=idx, max_seqlen=max_len, validated_metadata=ticket, fuse_many_rows=True)
    else:
        xr, xw, xk, xv, xa, xg = F.infer_tmix_mix6_forward_varlen(x, *mix, shift_state_pool=shift, cu_seqlens=cu,
                                                                  state_indices=idx, max_seqlen=max_len,
                                                                  validated_metadata=ticket)
        r = F.infer_tmix_linear_forward_varlen(xr, W["Wr"])
        k = F.infer_tmix_linear_forward_varlen(xk, W["Wk"])
        v = F.infer_tmix_linear_forward_varlen(xv, W["Wv"])
        fw, fa, fg, fv = F.infer_tmix_lowrank_wagv_in_forward_varlen(xw, xa, xg, xv, w1["w"], w1["a"], w1["g"], w1["v"])
    w, a12, gate, vres = F.infer_tmix_lowrank_vres_forward_varlen(fw, fa, fg, fv, w2["w"], w2["a"], w2["g"], w2["v"], v,
                                                                  v_first, W["v0"])
    kk, nkk, kka = F.infer_tmix_kk_a_gate_forward_varlen(k, W["k_k"], W["a0"], a12, W["k_a"], head_size=D,
                                                         batch_size=idx.numel(), max_seqlen=max_len)
    sh = (M, H, D)
    y = F.infer_recurrent_fp32io16_forward_varlen(r.view(sh), w.view(sh), kk.view(sh), vres.view(sh), nkk.view(sh),
                                                  kka.view(sh), state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                  validated_metadata=ticket, max_seqlen=max_len)
    z = F.infer_tmix_lnx_rkvres_xg_forward_varlen(y.view(M, C), r, kk, vres, W["r_k"], W["lnw"], W["lnb"], gate,
                                                  head_size=D, batch_size=idx.numel(), max_seqlen=max_len)
    return F.infer_tmix_linear_forward_varlen(z, W["Wo"])


CASES = [(D, M) for D in (64, 128, 256) for M in (1, 4, 7)] + [(64, 512), (128, 512)]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("packing", ["decode", "prefill"])
@pytest.mark.parametrize("D,M", CASES)
def test_layer_chain_matches_oracle_chain(oracle, D, M, packing, dtype):
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    H = C // D
    W = _weights(dtype, seed=1000 + D)
    gen = torch.Generator().manual_seed(M * 7 + D)
    x = torch.randn(M, C, generator=gen).to(dtype)
    v_first = torch.randn(M, C, generator=gen).to(dtype)
    if packing == "decode":
        cu = torch.arange(M + 1, dtype=torch.int32)
        idx = torch.randperm(M + 2, generator=gen)[:M].to(torch.int32)
    else:
        cu = torch.tensor([0, M], dtype=torch.int32)
        idx = torch.tensor([1], dtype=torch.int32)
    slots = int(idx.max()) + 2
    shift0 = torch.randn(slots, C, generator=gen).to(dtype)
    pool0 = synthetic.state_pool(slots, H, D, seed=D + M)
    want_out, want_pool, want_shift = _expected(oracle, W, x, v_first, shift0, pool0, cu, idx, D, dtype)

    dev = lambda t: t.cuda()  # noqa: E731
    Wd = {k: ({n: dev(t) for n, t in v.items()} if isinstance(v, dict) else [dev(t) for t in v] if isinstance(v, list)
              else dev(v)) for k, v in W.items()}
    bar_out, bar_state = (4e-3, 2e-3) if dtype == torch.float16 else (2.5e-2, 1e-2)
    for fused in (False, True):
        shift, pool = dev(shift0).clone(), dev(pool0).clone()
        out = _layer(F, Wd, dev(x), dev(v_first), shift, pool, dev(cu), dev(idx), D, fused)
        torch.cuda.synchronize()
        assert out.dtype == dtype and out.shape == (M, C)
        assert rel_rmse(out.float().cpu(), want_out) <= bar_out, (fused, rel_rmse(out.float().cpu(), want_out))
        assert rel_rmse(pool.cpu(), want_pool) <= bar_state, (fused, rel_rmse(pool.cpu(), want_pool))
        assert torch.equal(shift.cpu().float(), torch.as_tensor(want_shift).to(dtype).float())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("M", [1, 2, 4, 7, 8])
def test_one_launch_decode_layer_matches_oracle_chain_and_operator_sequence(oracle, M, dtype):
    """The persistent single-launch layer (grid-wide barriers between its stages) against the oracle chain, and
    against the operator sequence it replaces: same rounding points, so the two GPU paths differ by summation order
    only; scattered slots, untouched slots stay bit-identical, a second launch (the barrier counters must have been
    left at zero) and a CUDA-graph replay give the first launch's bits."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.tmix.layer import TMixLayerWeights, decode_layer_error_flag, reference_sequence

    D, H = 64, C // 64
    W = _weights(dtype, seed=2000 + M)
    gen = torch.Generator().manual_seed(M * 11)
    x = torch.randn(M, C, generator=gen).to(dtype)
    v_first = torch.randn(M, C, generator=gen).to(dtype)
    cu = torch.arange(M + 1, dtype=torch.int32)
    idx = torch.randperm(M + 3, generator=gen)[:M].to(torch.int32)
    slots = M + 3
    shift0 = torch.randn(slots, C, generator=gen).to(dtype)
    pool0 = synthetic.state_pool(slots, H, D, seed=M)
    want_out, want_pool, want_shift = _expected(oracle, W, x, v_first, shift0, pool0, cu, idx, D, dtype)
    d = lambda t: t.cuda()  # noqa: E731
    lw = TMixLayerWeights(*(d(m) for m in W["mix"]), d(W["Wr"]), d(W["Wk"]), d(W["Wv"]), d(W["Wo"]),
                          {n: d(t) for n, t in W["w1"].items()}, {n: d(t) for n, t in W["w2"].items()}, d(W["k_k"]),
                          d(W["a0"]), d(W["k_a"]), d(W["r_k"]), d(W["lnw"]), d(W["lnb"]), d(W["v0"]))
    # TMixLayerWeights takes the mix vectors in the order r, w, k, v, a, g: the order of W["mix"]
    bar_out, bar_state = (4e-3, 2e-3) if dtype == torch.float16 else (2.5e-2, 1e-2)
    shift, pool = d(shift0).clone(), d(pool0).clone()
    out = F.infer_tmix_decode_layer_forward_varlen(d(x), d(v_first), lw, shift_state_pool=shift, state_pool=pool,
                                                   cu_seqlens=d(cu), state_indices=d(idx))
    torch.cuda.synchronize()
    assert decode_layer_error_flag() == 0
    assert out.dtype == dtype and out.shape == (M, C)
    assert rel_rmse(out.float().cpu(), want_out) <= bar_out
    assert rel_rmse(pool.cpu(), want_pool) <= bar_state
    assert torch.equal(shift.cpu().float(), torch.as_tensor(want_shift).to(dtype).float())
    untouched = [s for s in range(slots) if s not in idx.tolist()]
    assert torch.equal(pool[untouched].cpu(), pool0[untouched])
    # the operator sequence on the same inputs
    shift_b, pool_b = d(shift0).clone(), d(pool0).clone()
    seq = reference_sequence(d(x), d(v_first), lw, shift_state_pool=shift_b, state_pool=pool_b, cu_seqlens=d(cu),
                             state_indices=d(idx))
    assert rel_rmse(out.float().cpu(), seq.float().cpu()) <= (2e-3 if dtype == torch.float16 else 1.2e-2)
    assert rel_rmse(pool.cpu(), pool_b.cpu()) <= (5e-4 if dtype == torch.float16 else 4e-3)
    assert torch.equal(shift, shift_b)
    # again, with a prepared ticket, eagerly and from a CUDA graph: the same bits as the first launch
    cu_d, idx_d, x_d, vf_d = d(cu), d(idx), d(x), d(v_first)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ticket = F.prepare_recurrent_metadata(cu_d, idx_d, total_tokens=M, state_pool_size=slots, max_seqlen=1)
        shift_c, pool_c = d(shift0).clone(), d(pool0).clone()
        run = lambda: F.infer_tmix_decode_layer_forward_varlen(  # noqa: E731
            x_d, vf_d, lw, shift_state_pool=shift_c, state_pool=pool_c, cu_seqlens=cu_d, state_indices=idx_d,
            validated_metadata=ticket)
        out_c = run()
        side.synchronize()
        assert torch.equal(out_c, out) and torch.equal(pool_c, pool)
        graph = torch.cuda.CUDAGraph()
        shift_c.copy_(d(shift0)); pool_c.copy_(d(pool0))
        with torch.cuda.graph(graph, stream=side):
            out_g = run()
        shift_c.copy_(d(shift0)); pool_c.copy_(d(pool0))
        graph.replay()
        side.synchronize()
        assert torch.equal(out_g, out) and torch.equal(pool_c, pool)
    torch.cuda.current_stream().wait_stream(side)
    assert decode_layer_error_flag() == 0
