"""Parity of the CUDA recurrence (through the public operator and the C ABI) with the CPU oracle.

Tolerances.  On identical 16-bit-rounded inputs the unrounded fp32 output must be
within 2e-2 max-abs of the float64 oracle and the final state within 1e-3 relative
error (the stated parity bar); the reference's own criterion, relative RMSE <= 2e-3
for output and state (tests/fixtures/tolerances-v1.json:9-12 of the reference), is
checked on the 16-bit output.
"""
import ctypes

import numpy as np
import pytest
import torch

from _util import load_golden, max_abs, rel_rmse

pytestmark = pytest.mark.gpu

TOKENS = ("r", "w", "k", "v", "a", "b")
Y_MAX_ABS = 2e-2
STATE_REL = 1e-3
REF_RMSE = 2e-3


def _dev(x):
    return x.cuda() if isinstance(x, torch.Tensor) else x


def _state_rel(actual, expected):
    e = torch.as_tensor(expected).double()
    a = torch.as_tensor(actual).double().cpu()
    return float((a - e).norm() / e.norm().clamp_min(1e-30))


def _run_public(g, **kw):
    import flashrwkv_b200 as F

    toks = [_dev(g[n]) for n in TOKENS]
    pool = _dev(g["state_pool"]).clone()
    y32 = torch.empty(toks[0].shape, device="cuda", dtype=torch.float32)
    bias = g.get("decay_bias")
    y = F.infer_recurrent_fp32io16_forward_varlen(
        *toks, state_pool=pool, cu_seqlens=_dev(g["cu_seqlens"]), state_indices=_dev(g["state_indices"]),
        scale=g.get("scale", 1.0), decay_bias=None if bias is None else _dev(bias), output_fp32=y32, **kw)
    torch.cuda.synchronize()
    return y, y32, pool


@pytest.mark.parametrize("name", ["recurrent_ragged", "rl_fp16"])
def test_golden_vectors_from_reference_oracle(name):
    g = load_golden(name)
    y, y32, pool = _run_public(g)
    assert max_abs(y32.cpu(), g["y"].float()) <= (Y_MAX_ABS if name == "recurrent_ragged" else 2e-3)
    assert rel_rmse(y.float().cpu(), g["y"].float()) <= REF_RMSE
    assert rel_rmse(pool.cpu(), g["final_pool"]) <= REF_RMSE
    assert _state_rel(pool, g["final_pool"]) <= STATE_REL
    # the 16-bit output is the correctly rounded fp32 output
    assert torch.equal(y, y32.to(y.dtype))
    # slots no sequence selects are bit-identical, selected ones changed
    active = set(g["state_indices"].tolist())
    before = g["state_pool"]
    for slot in range(before.shape[0]):
        same = torch.equal(pool[slot].cpu(), before[slot])
        assert same == (slot not in active)
    # determinism: a second run is bit-identical
    y_b, _, pool_b = _run_public(g)
    assert torch.equal(y, y_b) and torch.equal(pool, pool_b)


def test_cfg0_distribution_bf16_inputs_vs_oracle(oracle):
    g = load_golden("recurrent_cfg0")
    g16 = dict(g)
    for n in TOKENS:
        g16[n] = g[n].to(torch.bfloat16)
    y, y32, pool = _run_public(g16)
    ref = oracle.forward(*(g16[n] for n in TOKENS), state_pool=g["state_pool"], cu_seqlens=g["cu_seqlens"],
                         state_indices=g["state_indices"])
    assert max_abs(y32.cpu(), ref["y"]) <= Y_MAX_ABS
    assert _state_rel(pool, ref["state_pool"]) <= STATE_REL
    assert rel_rmse(y.float().cpu(), ref["y"]) <= REF_RMSE
    # against the golden (fp32-input) vector only input rounding separates the two
    assert rel_rmse(y32.cpu(), g["y"]) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_steps_at_benchmark_width(oracle, dtype):
    """B=256, H=32, D=64, one token per sequence, four consecutive in-place steps."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    B, H, D, steps = 256, 32, 64, 4
    cu, idx = synthetic.equal_length_metadata(B, 1)
    pool = synthetic.state_pool(B, H, D, seed=7)
    pool_dev = pool.cuda()
    ref_pool = pool.numpy()
    ticket = F.prepare_recurrent_metadata(cu.cuda(), idx.cuda(), total_tokens=B, state_pool_size=B)
    cu_d, idx_d = cu.cuda(), idx.cuda()
    ticket = F.prepare_recurrent_metadata(cu_d, idx_d, total_tokens=B, state_pool_size=B, max_seqlen=1)
    for step in range(steps):
        toks = synthetic.wkv7_inputs(B, H, D, seed=100 + step, dtype=dtype)
        y32 = torch.empty((B, H, D), device="cuda")
        y = F.infer_recurrent_fp32io16_forward_varlen(*(t.cuda() for t in toks), state_pool=pool_dev,
                                                      cu_seqlens=cu_d, state_indices=idx_d,
                                                      validated_metadata=ticket, max_seqlen=1, output_fp32=y32)
        ref = oracle.forward(*toks, state_pool=ref_pool, cu_seqlens=cu, state_indices=idx)
        ref_pool = ref["state_pool"]
        assert max_abs(y32.cpu(), ref["y"]) <= Y_MAX_ABS
        assert rel_rmse(y.float().cpu(), ref["y"]) <= REF_RMSE
    assert _state_rel(pool_dev, ref_pool) <= STATE_REL


def test_long_sequence_error_growth(oracle):
    from flashrwkv_b200 import synthetic

    B, T, H, D = 2, 512, 3, 64
    toks = synthetic.wkv7_inputs(B * T, H, D, seed=11)
    cu, idx = synthetic.equal_length_metadata(B, T)
    g = dict(zip(TOKENS, toks), cu_seqlens=cu, state_indices=idx, state_pool=synthetic.state_pool(B, H, D, seed=3))
    y, y32, pool = _run_public(g)
    ref = oracle.forward(*toks, state_pool=g["state_pool"], cu_seqlens=cu, state_indices=idx)
    assert max_abs(y32.cpu(), ref["y"]) <= Y_MAX_ABS
    assert _state_rel(pool, ref["state_pool"]) <= STATE_REL


def test_c_abi_direct_call_matches_operator():
    """Calls frwkv_wkv7_recurrent_fp32io16_forward_varlen through ctypes with raw pointers."""
    from flashrwkv_b200 import _ext

    lib = _ext.capi()
    g = load_golden("recurrent_ragged")
    y_op, _, pool_op = _run_public(g)
    toks = [_dev(g[n]) for n in TOKENS]
    pool = _dev(g["state_pool"]).clone()
    cu, idx = _dev(g["cu_seqlens"]), _dev(g["state_indices"])
    bias = _dev(g["decay_bias"])
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    cu_s, idx_s = torch.empty_like(cu), torch.empty_like(idx)
    N, H, D = toks[0].shape
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.frwkv_validate_recurrent_metadata(p(cu), p(idx), idx.numel(), N, pool.shape[0], p(status), p(cu_s),
                                               p(idx_s), stream)
    assert rc == 0, lib.frwkv_last_error()
    y = torch.empty_like(toks[3])
    rc = lib.frwkv_wkv7_recurrent_fp32io16_forward_varlen(
        p(cu_s), p(idx_s), p(status), p(pool), *(p(t) for t in toks), p(bias), p(y), None, N, idx.numel(), H, D,
        -1, 1, ctypes.c_float(g["scale"]), stream)
    assert rc == 0, lib.frwkv_last_error()
    torch.cuda.synchronize()
    assert status.tolist() == [0, 65]
    assert torch.equal(y, y_op) and torch.equal(pool, pool_op)
    # unsupported head size and null pointers are refused with a message, nothing is launched
    rc = lib.frwkv_wkv7_recurrent_fp32io16_forward_varlen(
        p(cu_s), p(idx_s), p(status), p(pool), *(p(t) for t in toks), None, p(y), None, N, idx.numel(), H, 96,
        -1, 1, ctypes.c_float(1.0), stream)
    assert rc == -2 and b"head size" in lib.frwkv_last_error()
    rc = lib.frwkv_wkv7_recurrent_fp32io16_forward_varlen(
        None, p(idx_s), p(status), p(pool), *(p(t) for t in toks), None, p(y), None, N, idx.numel(), H, D,
        -1, 1, ctypes.c_float(1.0), stream)
    assert rc == -1


BAD_METADATA = ["wrong_rank", "wrong_length", "wrong_dtype", "wrong_start", "wrong_end", "non_increasing",
                "wrong_slot_length", "duplicate_slot", "negative_slot", "out_of_range_slot"]


@pytest.mark.parametrize("kind", BAD_METADATA)
def test_invalid_metadata_raises_and_preserves_state(kind):
    import flashrwkv_b200 as F

    g = load_golden("recurrent_ragged")
    toks = [_dev(g[n]) for n in TOKENS]
    pool = _dev(g["state_pool"]).clone()
    cu, idx = _dev(g["cu_seqlens"]), _dev(g["state_indices"])
    if kind == "wrong_rank":
        cu = cu.reshape(1, -1)
    elif kind == "wrong_length":
        cu = cu[:-1]
    elif kind == "wrong_dtype":
        cu = cu.to(torch.int64)
    elif kind == "wrong_start":
        cu = cu + 1
    elif kind == "wrong_end":
        cu = cu.clone()
        cu[-1] -= 1
    elif kind == "non_increasing":
        cu = cu.clone()
        cu[2] = cu[1]
    elif kind == "wrong_slot_length":
        idx = idx[:-1]
    elif kind == "duplicate_slot":
        idx = idx.clone()
        idx[1] = idx[0]
    elif kind == "negative_slot":
        idx = idx.clone()
        idx[0] = -1
    else:
        idx = idx.clone()
        idx[0] = pool.shape[0]
    before = pool.clone()
    with pytest.raises((TypeError, ValueError, RuntimeError)):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx)
    torch.cuda.synchronize()
    assert torch.equal(pool, before)


def test_low_level_call_with_bad_metadata_fails_closed():
    from flashrwkv_b200 import _ext

    C = _ext.extension()
    toks = [(torch.randn(4, 2, 64, device="cuda") * 0.1).half() for _ in range(6)]
    pool = torch.randn(3, 2, 64, 64, device="cuda")
    before = pool.clone()
    out = torch.zeros_like(toks[3])
    C.recurrent_fp32_from_decay_logits(torch.tensor([1, 4], device="cuda", dtype=torch.int32),
                                       torch.tensor([0], device="cuda", dtype=torch.int32), pool, *toks, out, 1.0,
                                       None, None)
    torch.cuda.synchronize()
    assert torch.isnan(out).all()
    assert torch.equal(pool, before)


def test_ticket_mismatches_and_structural_rejections():
    import flashrwkv_b200 as F

    g = load_golden("recurrent_ragged")
    toks = [_dev(g[n]) for n in TOKENS]
    pool = _dev(g["state_pool"]).clone()
    cu, idx = _dev(g["cu_seqlens"]), _dev(g["state_indices"])
    kw = dict(state_pool=pool, cu_seqlens=cu, state_indices=idx)
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=toks[0].shape[0], state_pool_size=pool.shape[0])
    with pytest.raises(RuntimeError, match="identity"):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu.clone(), state_indices=idx,
                                                  validated_metadata=ticket)
    with pytest.raises(RuntimeError, match="total_tokens"):
        F.infer_recurrent_fp32io16_forward_varlen(*(t[:-1].contiguous() for t in toks), **kw,
                                                  validated_metadata=ticket)
    with pytest.raises(RuntimeError, match="state_pool_size"):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=torch.cat((pool, pool[:1])), cu_seqlens=cu,
                                                  state_indices=idx, validated_metadata=ticket)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with pytest.raises(RuntimeError, match="stream"):
            F.infer_recurrent_fp32io16_forward_varlen(*toks, **kw, validated_metadata=ticket)
    side.synchronize()
    cu[1] += 1
    with pytest.raises(RuntimeError, match="version"):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, **kw, validated_metadata=ticket)
    cu[1] -= 1
    # structural rejections before any launch
    with pytest.raises(ValueError, match="contiguous"):
        F.infer_recurrent_fp32io16_forward_varlen(toks[0].transpose(0, 1), *toks[1:], **kw)
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        F.infer_recurrent_fp32io16_forward_varlen(*(t.float() for t in toks), **kw)
    with pytest.raises(RuntimeError, match="dtype mismatch"):
        F.infer_recurrent_fp32io16_forward_varlen(toks[0], toks[1].half(), *toks[2:], **kw)
    with pytest.raises(TypeError, match="float32"):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool.half(), cu_seqlens=cu, state_indices=idx)
    with pytest.raises(RuntimeError, match="square"):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool[..., :-1].contiguous(), cu_seqlens=cu,
                                                  state_indices=idx)
    with pytest.raises(RuntimeError, match="finite"):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, **kw, scale=float("nan"))
    with pytest.raises((ValueError, RuntimeError), match="decay_bias"):
        F.infer_recurrent_fp32io16_forward_varlen(*toks, **kw, decay_bias=torch.zeros(2, 63, device="cuda",
                                                                                      dtype=toks[0].dtype))


def test_cuda_graph_replay_with_ticket(oracle):
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    B, H, D = 8, 4, 64
    toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=5)]
    cu, idx = (t.cuda() for t in synthetic.equal_length_metadata(B, 1))
    pool0 = synthetic.state_pool(B, H, D, seed=6)
    pool = pool0.cuda()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B)
        F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool.clone(), cu_seqlens=cu, state_indices=idx,
                                                  validated_metadata=ticket)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y = F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                          validated_metadata=ticket)
        graph.replay()
        graph.replay()
    side.synchronize()
    ref_pool = pool0.numpy()
    for _ in range(2):
        ref = oracle.forward(*toks, state_pool=ref_pool, cu_seqlens=cu, state_indices=idx)
        ref_pool = ref["state_pool"]
    assert rel_rmse(y.float().cpu(), ref["y"]) <= REF_RMSE
    assert _state_rel(pool, ref_pool) <= STATE_REL


def test_host_decode_loop_is_bit_identical_to_serial_decode():
    """The three-stream host loop (pinned inputs in, pinned outputs out) gives the serial result, step by step."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic
    from flashrwkv_b200.host_io import HostDecodeLoop

    B, H, D, steps = 48, 4, 64, 9
    cu, idx = (t.cuda() for t in synthetic.equal_length_metadata(B, 1))
    pool_a = synthetic.state_pool(B, H, D, seed=5, device="cuda")
    pool_b = pool_a.clone()
    host = [[t.pin_memory() for t in synthetic.wkv7_inputs(B, H, D, seed=100 + i)] for i in range(steps)]
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B, max_seqlen=1)
    loop = HostDecodeLoop(host[0], state_pool=pool_a, cu_seqlens=cu, state_indices=idx, validated_metadata=ticket)
    outs = [torch.empty((B, H, D), dtype=torch.bfloat16).pin_memory() for _ in range(steps)]
    for i in range(steps):
        # six separate pinned tensors on even steps, one packed pinned buffer on odd ones
        loop.submit(host[i] if i % 2 == 0 else torch.stack(host[i]).pin_memory(), outs[i])
    loop.drain()
    torch.cuda.synchronize()
    for i in range(steps):
        y = F.infer_recurrent_fp32io16_forward_varlen(*[t.cuda() for t in host[i]], state_pool=pool_b, cu_seqlens=cu,
                                                      state_indices=idx, validated_metadata=ticket, max_seqlen=1)
        assert torch.equal(y.cpu(), outs[i]), f"step {i}"
    assert torch.equal(pool_a, pool_b)
    with pytest.raises(ValueError):
        HostDecodeLoop([t.cuda() for t in host[0]], state_pool=pool_a, cu_seqlens=cu, state_indices=idx,
                       validated_metadata=ticket)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [128, 256])
def test_head_sizes_128_and_256_vs_oracle(oracle, D, dtype):
    """The general kernel for the reference's other head sizes: ragged batch, slot selection, bias, scale."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    H, lengths, slots = 2, (1, 9, 33), 5
    N = sum(lengths)
    toks = [t.to(dtype) for t in synthetic.wkv7_inputs(N, H, D, seed=900 + D, dtype=torch.float32)]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32)
    idx = torch.tensor([4, 0, 2], dtype=torch.int32)
    gen = torch.Generator().manual_seed(D)
    pool = torch.randn(slots, H, D, D, generator=gen) * 0.05
    bias = (torch.randn(H, D, generator=gen) * 0.2).to(dtype)
    d_pool = pool.cuda()
    y32 = torch.empty(N, H, D, device="cuda")
    y = F.infer_recurrent_fp32io16_forward_varlen(*[t.cuda() for t in toks], state_pool=d_pool, cu_seqlens=cu.cuda(),
                                                  state_indices=idx.cuda(), scale=0.5, decay_bias=bias.cuda(),
                                                  output_fp32=y32)
    torch.cuda.synchronize()
    ref = oracle.forward(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx, scale=0.5, decay_bias=bias)
    assert max_abs(y32.cpu(), ref["y"]) <= Y_MAX_ABS
    assert rel_rmse(y.float().cpu(), ref["y"]) <= REF_RMSE
    assert _state_rel(d_pool, ref["state_pool"]) <= STATE_REL
    assert torch.equal(y, y32.to(dtype))
    assert torch.equal(d_pool[[1, 3]].cpu(), pool[[1, 3]])


@pytest.mark.parametrize("B", [48, 160])  # 1536 tiles: the register kernel; 5120 tiles: the bulk-copy ring kernel
def test_wait_timeout_bit_in_the_status_word_fails_closed(B):
    """A decode kernel whose bounded wait ran out leaves FRWKV_META_WAIT_TIMEOUT (16) in the ticket's status word;
    from then on every call with that ticket must behave like a call with bad metadata: NaN outputs, pool untouched."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    H, D = 32, 64
    toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=3)]
    cu, idx = (t.cuda() for t in synthetic.equal_length_metadata(B, 1))
    pool = synthetic.state_pool(B, H, D, seed=4, device="cuda")
    ticket = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B, max_seqlen=1)
    y = F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                  validated_metadata=ticket, max_seqlen=1)
    torch.cuda.synchronize()
    assert int(ticket._status().item()) == 0 and torch.isfinite(y.float()).all()
    before = pool.clone()
    ticket._status().fill_(16)
    y = F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool, cu_seqlens=cu, state_indices=idx,
                                                  validated_metadata=ticket, max_seqlen=1)
    torch.cuda.synchronize()
    assert torch.isnan(y.float()).all()
    assert torch.equal(pool, before)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_direct_slot_decode_is_bit_identical_to_indexed_decode(dtype):
    """A ticket made from `cu_seqlens = 0..B` and `state_indices = 0..B-1` knows that sequence i is token i in slot i,
    and small decode batches then take a kernel that reads neither table.  The same tokens decoded through a shuffled
    slot table (which takes the indexed kernel) must give the same bits, outputs and states, over several steps."""
    import flashrwkv_b200 as F
    from flashrwkv_b200 import synthetic

    B, H, D, steps = 48, 32, 64, 3
    cu, idx = (t.cuda() for t in synthetic.equal_length_metadata(B, 1))
    perm = torch.randperm(B, generator=torch.Generator().manual_seed(5)).to(torch.int32).cuda()
    pool_a = synthetic.state_pool(B, H, D, seed=21, device="cuda")
    pool_b = torch.empty_like(pool_a)
    pool_b[perm.long()] = pool_a  # sequence i's state lives in slot perm[i]
    ticket_a = F.prepare_recurrent_metadata(cu, idx, total_tokens=B, state_pool_size=B, max_seqlen=1)
    ticket_b = F.prepare_recurrent_metadata(cu, perm, total_tokens=B, state_pool_size=B, max_seqlen=1)
    assert ticket_a._direct_slots() and not ticket_b._direct_slots()
    for step in range(steps):
        toks = [t.cuda() for t in synthetic.wkv7_inputs(B, H, D, seed=300 + step, dtype=dtype)]
        ya = F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool_a, cu_seqlens=cu, state_indices=idx,
                                                       validated_metadata=ticket_a, max_seqlen=1)
        yb = F.infer_recurrent_fp32io16_forward_varlen(*toks, state_pool=pool_b, cu_seqlens=cu, state_indices=perm,
                                                       validated_metadata=ticket_b, max_seqlen=1)
        assert torch.equal(ya, yb)
    assert torch.equal(pool_a, pool_b[perm.long()])
    # a batch that is not one token per sequence never gets the flag
    cu2 = torch.tensor([0, 2, 3], dtype=torch.int32, device="cuda")
    idx2 = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    assert not F.prepare_recurrent_metadata(cu2, idx2, total_tokens=3, state_pool_size=B)._direct_slots()
