"""Pins the CPU oracle against vectors produced by the reference's own test oracles."""
import numpy as np
import torch

from _util import load_golden, max_abs, rel_rmse

TOKENS = ("r", "w", "k", "v", "a", "b")


def _run(oracle, g, **kw):
    return oracle.forward(*(g[n] for n in TOKENS), state_pool=g["state_pool"], cu_seqlens=g["cu_seqlens"],
                          state_indices=g.get("state_indices"), scale=g.get("scale", 1.0),
                          decay_bias=g.get("decay_bias"), **kw)


def test_recurrent_cfg0_both_accumulators(oracle):
    g = load_golden("recurrent_cfg0")
    for double in (True, False):
        out = _run(oracle, g, double=double)
        assert max_abs(out["y"], g["y"]) < 2e-4
        assert rel_rmse(out["y"], g["y"]) < 2e-6
        assert rel_rmse(out["state_pool"], g["final_pool"]) < 2e-6


def test_recurrent_ragged_slots_bias_scale(oracle):
    g = load_golden("recurrent_ragged")
    out = _run(oracle, g)
    assert rel_rmse(out["y"], g["y"]) < 1e-6
    assert rel_rmse(out["state_pool"], g["final_pool"]) < 1e-6
    inactive = [1, 3, 6, 8]
    assert np.array_equal(out["state_pool"][inactive], g["state_pool"].numpy()[inactive])


def test_torch_restatement_matches_reference_oracle(oracle):
    g = load_golden("recurrent_ragged")
    y, pool = oracle.forward_torch(*(g[n] for n in TOKENS), state_pool=g["state_pool"],
                                   cu_seqlens=g["cu_seqlens"], state_indices=g["state_indices"],
                                   scale=g["scale"], decay_bias=g["decay_bias"])
    assert rel_rmse(y, g["y"]) < 1e-6
    assert rel_rmse(pool, g["final_pool"]) < 1e-6


def test_chunk_bf16_reference_rounds_outputs(oracle):
    g = load_golden("chunk_bf16")
    out = _run(oracle, g)
    y = torch.from_numpy(out["y"]).to(torch.bfloat16)
    # the reference oracle rounds y and the final state to bf16: allow one ulp of disagreement
    assert rel_rmse(y.float(), g["y"].float()) < 4e-3
    final = torch.from_numpy(out["state_pool"]).to(torch.bfloat16)
    assert rel_rmse(final.float(), g["final_pool"].float()) < 4e-3


def test_rl_fp16_io(oracle):
    g = load_golden("rl_fp16")
    out = _run(oracle, g)
    assert max_abs(torch.from_numpy(out["y"]).half().float(), g["y"].float()) <= 2e-6
    assert rel_rmse(out["state_pool"], g["final_pool"]) < 1e-6


def test_statetune_outputs_and_gradients(oracle):
    g = load_golden("statetune")
    B = g["S0"].shape[0]
    chunks = (g["seq_chunk_offsets"], g["chunk_starts"], g["chunk_ends"])
    cu = torch.tensor([0, 3, 5], dtype=torch.int32)  # token ranges implied by the chunk tables
    out = oracle.forward(*(g[n] for n in TOKENS), state_pool=g["S0"], cu_seqlens=cu,
                         state_indices=torch.arange(B, dtype=torch.int32), scale=g["scale"],
                         chunks=chunks, want_state_dot_a=True)
    assert max_abs(torch.from_numpy(out["y"]).half().float(), g["y"].float()) <= 2e-7
    assert rel_rmse(out["state_pool"], g["final_state"]) < 1e-6
    assert rel_rmse(out["boundary"], g["boundary"]) < 1e-6
    assert rel_rmse(out["state_dot_a"], g["state_dot_a"]) < 1e-5
    grads = oracle.backward(*(g[n] for n in TOKENS), initial_state=g["S0"], cu_seqlens=cu,
                            grad_output=g["grad_output"], grad_final_state=g["grad_final_state"],
                            scale=g["scale"])
    for ours, name in (("initial_state", "dS0"), ("r", "dr"), ("decay_logits", "dw"), ("k", "dk"),
                       ("v", "dv"), ("a", "da"), ("b", "db")):
        assert torch.allclose(torch.from_numpy(grads[ours]), g[name], atol=3e-6, rtol=3e-3), name


def test_pretrain_dense_forward_and_gradients(oracle):
    g = load_golden("pretrain")
    Bp, Tp, C = g["r"].shape
    H, D = C // 64, 64
    toks = [g[n].reshape(Bp * Tp, H, D) for n in TOKENS]
    cu = torch.arange(Bp + 1, dtype=torch.int32) * Tp
    S0 = torch.zeros(Bp, H, D, D)
    out = oracle.forward(*toks, state_pool=S0, cu_seqlens=cu)
    assert rel_rmse(out["y"].reshape(Bp, Tp, C), g["y"]) < 1e-5
    grads = oracle.backward(*toks, initial_state=S0, cu_seqlens=cu,
                            grad_output=g["dy"].reshape(Bp * Tp, H, D))
    for ours, name in (("r", "dr"), ("decay_logits", "dw"), ("k", "dk"), ("v", "dv"), ("a", "da"), ("b", "db")):
        # the reference's autograd leaves are bf16, so its gradients carry one bf16 rounding
        assert rel_rmse(grads[ours].reshape(Bp, Tp, C), g[name]) < 4e-3, name


def test_retention_matches_exp2_form(oracle):
    x = np.linspace(-12, 14, 4001, dtype=np.float32)
    w = oracle.retention(x)
    ref = np.exp2(-0.8750387749145276 / (1.0 + np.exp2(-1.4426950408889634 * x.astype(np.float64))))
    assert np.max(np.abs(w - ref)) < 2e-7
    assert w.min() > 0.545 and w.max() < 1.0


def test_tmix_pieces_match_reference_formulas(oracle):
    g = load_golden("tmix_kk_a_gate")
    outs = oracle.kk_a_gate(g["k"], g["k_k"], g["a0"], g["a12"], g["k_a"])
    for ours, name in zip(outs, ("new_k", "neg_kk", "kka")):
        assert max_abs(ours, g[name]) < 1e-5, name
    g = load_golden("tmix_lnx")
    out = oracle.lnx_rkvres_xg(g["x"], g["r"], g["k"], g["v"], g["r_k"], g["weight"], g["bias"], g["g"])
    assert rel_rmse(out, g["out"]) < 1e-6
    g = load_golden("tmix_vres")
    assert max_abs(oracle.vres_gate(g["v"], g["v_first"], g["v0"], g["v12"]), g["out"]) < 1e-6
    g = load_golden("tmix_mix6")
    out, shift = oracle.mix6(g["x"], g["shift_pool"], list(g["mix"]), g["cu_seqlens"], g["state_indices"])
    assert max_abs(out, g["out"]) < 1e-5
    assert np.array_equal(shift, g["shift_after"].float().numpy())
    g = load_golden("tmix_lowrank")
    rank = oracle.linear_nt(g["x"], g["w1"])
    assert max_abs(torch.from_numpy(rank).half().float(), g["rank"].float()) < 2e-3
    assert rel_rmse(oracle.linear_nt(g["rank"], g["w2"], act="tanh"), g["out_tanh"]) < 1e-6
    # closed-form answer pinned by the reference (tests/tmix/kk_a_gate/test.py:45-47): all-ones inputs, C = 4096
    ones = np.ones((2, 4096), np.float32)
    new_k, neg_kk, kka = oracle.kk_a_gate(ones, ones[0], 0 * ones[0], 0 * ones, ones[0])
    assert np.allclose(new_k, 0.5) and np.allclose(neg_kk, -0.125) and np.allclose(kka, 0.0625)


def test_fp16_state_contract_with_dither(oracle):
    """The fp16-state restatement follows the reference oracle through rounding: values that differ at all differ
    by one fp16 ulp (a tie broken the other way by a last-bit difference in exp / sigmoid), and few do."""
    g = load_golden("recurrent_fp16state")
    out = oracle.forward_fp16(*(g[n] for n in TOKENS), state_pool=g["state_pool"],
                              elapsed_state_pool=g["elapsed_state_pool"], cu_seqlens=g["cu_seqlens"],
                              state_indices=g["state_indices"], scale=g["scale"], decay_bias=g["decay_bias"])
    got_state = torch.from_numpy(out["state_pool"])
    want_state = g["final_pool"]
    assert got_state.dtype == torch.float16 and want_state.dtype == torch.float16
    mismatch = (got_state != want_state).float().mean().item()
    assert mismatch < 2e-3
    assert rel_rmse(got_state.float(), want_state.float()) < 2e-4
    assert rel_rmse(out["y"], g["y"].float()) < 2e-4
    inactive = [1, 3, 6, 8]
    assert torch.equal(got_state[inactive], g["state_pool"][inactive])
    # the dither phase matters: other elapsed counters give a different rounded state
    shifted = oracle.forward_fp16(*(g[n] for n in TOKENS), state_pool=g["state_pool"],
                                  elapsed_state_pool=g["elapsed_state_pool"] + 1, cu_seqlens=g["cu_seqlens"],
                                  state_indices=g["state_indices"], scale=g["scale"], decay_bias=g["decay_bias"])
    assert (torch.from_numpy(shifted["state_pool"]) != want_state).float().mean().item() > 1e-2


def test_fp16_state_contract_head_size_128(oracle):
    """The same contract at head size 128 (the dither phase runs over head * 128 + channel)."""
    g = load_golden("recurrent_fp16state_d128")
    out = oracle.forward_fp16(*(g[n] for n in TOKENS), state_pool=g["state_pool"],
                              elapsed_state_pool=g["elapsed_state_pool"], cu_seqlens=g["cu_seqlens"],
                              state_indices=g["state_indices"], scale=g["scale"], decay_bias=g["decay_bias"])
    got_state, want_state = torch.from_numpy(out["state_pool"]), g["final_pool"]
    assert (got_state != want_state).float().mean().item() < 2e-3
    assert rel_rmse(got_state.float(), want_state.float()) < 2e-4
    assert rel_rmse(out["y"], g["y"].float()) < 2e-4
    assert torch.equal(got_state[[1]], g["state_pool"][[1]])


def test_layer_norm_family_formulas(oracle):
    g = load_golden("tmix_norm")
    assert rel_rmse(oracle.layer_norm(g["x"], g["weight"], g["bias"]), g["ln_x"]) < 1e-5
    summed, normed = oracle.layer_norm(g["x"], g["weight"], g["bias"], residual=g["residual"], io_dtype=torch.float16)
    assert np.array_equal(summed, g["sum"].float().numpy())
    assert rel_rmse(normed, g["ln_sum"]) < 1e-5
