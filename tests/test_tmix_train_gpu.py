"""Parity of the training-side TMix operators (forward and backward through autograd) with the float64 oracle.

The kernels compute in fp32 and round once to bf16, and so does the reference; every tensor must therefore be the
oracle's value up to one bf16 rounding (relative RMSE <= 4e-3).  Parameter gradients are fp32 sums over the B*T rows
rounded once, same bound.  Shapes: the reference tests' own (B=2, T=3, C=2*head_size; mix6 with C=8) and a larger one
whose rows fall into many slabs with sequence boundaries inside slabs and two channel tiles.
"""
import pytest
import torch

from _util import rel_rmse

pytestmark = pytest.mark.gpu

TOL = 4e-3
SHAPES = [(2, 3, None), (3, 131, 2048)]  # C = None: two heads


def _rn(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16).cuda().requires_grad_()


def _check(got, want, name):
    got = got.detach().float().cpu()
    assert torch.isfinite(got).all(), name
    assert rel_rmse(got, torch.from_numpy(want).float()) <= TOL, name


@pytest.mark.parametrize("B,T,C", [(2, 3, 16), (3, 131, 2048), (1, 1, 8)])
def test_a_gate_and_vres_gate(B, T, C):
    import flashrwkv_b200 as F
    from oracle import tmix_train_oracle as O

    gen = torch.Generator().manual_seed(B * 1000 + T)
    a0, a12, go = _rn(gen, C), _rn(gen, B, T, C), _rn(gen, B, T, C)
    y = F.pretrain_tmix_a_gate_bf16(a0, a12)
    _check(y, O.a_gate(a0, a12), "a_gate")
    y.backward(go)
    for got, want, name in zip((a0.grad, a12.grad), O.a_gate_backward(go, a0, a12), ("d a0", "d a12")):
        _check(got, want, name)
    v, vf, v0, v12 = _rn(gen, B, T, C), _rn(gen, B, T, C), _rn(gen, C), _rn(gen, B, T, C)
    y = F.pretrain_tmix_vres_gate_bf16(v, vf, v0, v12)
    _check(y, O.vres_gate(v, vf, v0, v12), "vres_gate")
    y.backward(go)
    for got, want, name in zip((v.grad, vf.grad, v0.grad, v12.grad), O.vres_gate_backward(go, v, vf, v0, v12),
                               ("d v", "d v_first", "d v0", "d v12")):
        _check(got, want, name)


@pytest.mark.parametrize("B,T,C", [(2, 3, 8), (3, 131, 2048), (5, 1, 64), (1, 700, 1032)])
def test_mix6(B, T, C):
    import flashrwkv_b200 as F
    from oracle import tmix_train_oracle as O

    gen = torch.Generator().manual_seed(B * 1000 + T)
    x = _rn(gen, B, T, C, scale=0.1)
    mixes = [_rn(gen, C, scale=0.5) for _ in range(6)]
    gos = [_rn(gen, B, T, C) for _ in range(6)]
    outs = F.pretrain_tmix_mix6_bf16(x, *mixes)
    for j, (got, want) in enumerate(zip(outs, O.mix6(x, mixes))):
        _check(got, want, f"mix6 out {j}")
    torch.autograd.backward(outs, gos)
    gx, gm, _ = O.mix6_backward(gos, x, mixes)
    _check(x.grad, gx, "d x")
    for j in range(6):
        _check(mixes[j].grad, gm[j], f"d mix {j}")


@pytest.mark.parametrize("B,T,C", [(1, 1, 128), (2, 7, 128), (2, 31, 128), (3, 131, 2048)])
@pytest.mark.parametrize("zero_shift", [False, True])
def test_statetune_mix6(B, T, C, zero_shift):
    """Shapes of the reference's test (tests/tmix/mix6/test.py:88-135) plus one with many slabs; with a zero shift
    state the six outputs are bit-identical to the pretrain form's."""
    import flashrwkv_b200 as F
    from oracle import tmix_train_oracle as O

    gen = torch.Generator().manual_seed(1000 + B * 100 + T)
    x = _rn(gen, B, T, C, scale=0.05)
    initial = _rn(gen, B, C, scale=0.0 if zero_shift else 0.05)
    mixes = [_rn(gen, C, scale=0.1) for _ in range(6)]
    gos = [_rn(gen, B, T, C) for _ in range(6)] + [_rn(gen, B, C)]
    outs = F.statetune_tmix_mix6_bf16(x, initial, *mixes)
    assert len(outs) == 7
    for j, (got, want) in enumerate(zip(outs[:6], O.mix6(x, mixes, initial))):
        _check(got, want, f"mix6 out {j}")
    assert torch.equal(outs[6], x[:, -1, :])
    grads = torch.autograd.grad(outs, [x, initial, *mixes], gos)
    gx, gm, ginit = O.mix6_backward(gos[:6], x, mixes, initial, gos[6])
    _check(grads[0], gx, "d x")
    _check(grads[1], ginit, "d initial_shift")
    for j in range(6):
        _check(grads[2 + j], gm[j], f"d mix {j}")
    if zero_shift:
        for a, b in zip(outs[:6], F.pretrain_tmix_mix6_bf16(x.detach(), *(m.detach() for m in mixes))):
            assert torch.equal(a, b)


def test_statetune_mix6_chunk_composition():
    """Two chunks chained through the shift state give the whole sequence's outputs and gradients
    (tests/tmix/mix6/test.py:138-185)."""
    import flashrwkv_b200 as F

    gen = torch.Generator().manual_seed(23)
    B, T, C, split = 2, 7, 128, 3
    x, initial = _rn(gen, B, T, C), _rn(gen, B, C)
    mixes = [_rn(gen, C) for _ in range(6)]
    whole = F.statetune_tmix_mix6_bf16(x, initial, *mixes)
    ups = [_rn(gen, B, T, C).detach() for _ in range(6)] + [_rn(gen, B, C).detach()]
    whole_grads = torch.autograd.grad(whole, [x, initial, *mixes], ups)
    x2, init2 = x.detach().clone().requires_grad_(), initial.detach().clone().requires_grad_()
    mixes2 = [m.detach().clone().requires_grad_() for m in mixes]
    first = F.statetune_tmix_mix6_bf16(x2[:, :split].contiguous(), init2, *mixes2)
    second = F.statetune_tmix_mix6_bf16(x2[:, split:].contiguous(), first[6], *mixes2)
    for j in range(6):
        assert torch.equal(torch.cat((first[j], second[j]), dim=1), whole[j])
    assert torch.equal(second[6], whole[6])
    chained = [torch.cat((first[j], second[j]), dim=1) for j in range(6)] + [second[6]]
    grads2 = torch.autograd.grad(chained, [x2, init2, *mixes2], ups)
    for a, b in zip(whole_grads, grads2):
        assert torch.allclose(a.float(), b.float(), atol=0.03, rtol=0.03)


@pytest.mark.parametrize("head_size", [64, 128, 256])
@pytest.mark.parametrize("B,T,C", SHAPES)
def test_kk_pre(head_size, B, T, C):
    import flashrwkv_b200 as F
    from oracle import tmix_train_oracle as O

    C = C or 2 * head_size
    gen = torch.Generator().manual_seed(19 + head_size)
    k, k_k, a, k_a = _rn(gen, B, T, C, scale=0.1), _rn(gen, C, scale=0.1), _rn(gen, B, T, C, scale=0.1), _rn(gen, C)
    gos = [_rn(gen, B, T, C) for _ in range(3)]
    outs = F.pretrain_tmix_kk_pre_bf16(k, k_k, a, k_a, head_size=head_size)
    assert len(outs) == 3
    for got, want, name in zip(outs, O.kk_pre(k, k_k, a, k_a, head_size), ("new_k", "neg_kk", "kka")):
        _check(got, want, name)
    torch.autograd.backward(outs, gos)
    for got, want, name in zip((k.grad, k_k.grad, a.grad, k_a.grad),
                               O.kk_pre_backward(*gos, k, k_k, a, k_a, head_size), ("d k", "d k_k", "d a", "d k_a")):
        _check(got, want, name)


@pytest.mark.parametrize("head_size", [64, 128, 256])
@pytest.mark.parametrize("B,T,C", SHAPES)
def test_lnx_rkvres_xg(head_size, B, T, C):
    import flashrwkv_b200 as F
    from oracle import tmix_train_oracle as O

    C = C or 2 * head_size
    gen = torch.Generator().manual_seed(23 + head_size)
    x, r, k, v = (_rn(gen, B, T, C, scale=0.3) for _ in range(4))
    r_k, weight, bias = _rn(gen, C // head_size, head_size, scale=0.1), _rn(gen, C), _rn(gen, C)
    g, go = _rn(gen, B, T, C), _rn(gen, B, T, C)
    y = F.pretrain_tmix_lnx_rkvres_xg_bf16(x, r, k, v, r_k, weight, bias, g, head_size=head_size)
    assert y.shape == x.shape
    _check(y, O.lnx_rkvres_xg(x, r, k, v, r_k, weight, bias, g, head_size)[0], "lnx out")
    y.backward(go)
    want = O.lnx_rkvres_xg_backward(go, x, r, k, v, r_k, weight, bias, g, head_size)
    names = ("d x", "d r", "d k", "d v", "d r_k", "d weight", "d bias", "d g")
    for t, w, name in zip((x, r, k, v, r_k, weight, bias, g), want, names):
        assert t.grad.shape == t.shape
        _check(t.grad, w, name)


def test_zero_key_row_and_unused_outputs():
    """A zero key is below the normalisation clamp (no projection term, finite gradients); outputs that take no part
    in the loss get zero gradients."""
    import flashrwkv_b200 as F

    C = 128
    k = torch.zeros(1, 2, C, dtype=torch.bfloat16, device="cuda").requires_grad_()
    vec = torch.ones(C, dtype=torch.bfloat16, device="cuda").requires_grad_()
    a = torch.full((1, 2, C), 0.5, dtype=torch.bfloat16, device="cuda").requires_grad_()
    new_k, neg_kk, kka = F.pretrain_tmix_kk_pre_bf16(k, vec, a, vec)
    assert float(neg_kk.detach().float().abs().max()) == 0.0
    new_k.float().sum().backward()
    assert torch.isfinite(k.grad.float()).all() and torch.equal(k.grad.float(), a.detach().float())


def test_parameter_gradients_are_reproducible_and_api_refusals():
    import inspect

    import flashrwkv_b200 as F

    gen = torch.Generator().manual_seed(5)
    x = _rn(gen, 4, 512, 2048, scale=0.1)
    mixes = [_rn(gen, 2048) for _ in range(6)]
    gos = [_rn(gen, 4, 512, 2048) for _ in range(6)]
    runs = []
    for _ in range(2):
        outs = F.pretrain_tmix_mix6_bf16(x, *mixes)
        runs.append(torch.autograd.grad(outs, [x, *mixes], gos))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    assert inspect.signature(F.pretrain_tmix_kk_pre_bf16).parameters["head_size"].default == 64
    assert inspect.signature(F.pretrain_tmix_lnx_rkvres_xg_bf16).parameters["head_size"].default == 64
    key = torch.zeros(1, 1, 65, device="cuda", dtype=torch.bfloat16)
    vector = torch.zeros(65, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="divisible by head_size"):
        F.pretrain_tmix_kk_pre_bf16(key, vector, key, vector)
    with pytest.raises(ValueError, match="bfloat16"):
        F.pretrain_tmix_a_gate_bf16(vector.half(), key.half())
    with pytest.raises(ValueError, match=r"\[C\]"):
        F.pretrain_tmix_mix6_bf16(x.detach(), *[m.detach()[:8] for m in mixes])


def test_full_size_backward_is_linear_in_upstream_gradient():
    """B=8, T=4096, C=4096 (the training configuration's activations): grads(g1 + g2) = grads(g1) + grads(g2) up to
    the single bf16 rounding of each result."""
    import flashrwkv_b200 as F

    B, T, C = 8, 4096, 4096
    gen = torch.Generator(device="cuda").manual_seed(6)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=gen).to(torch.bfloat16)  # noqa: E731
    x, r, k, v, g = (rn(B, T, C).requires_grad_() for _ in range(5))
    r_k, weight, bias = (rn(C // 64, 64) * 0.1).requires_grad_(), rn(C).requires_grad_(), rn(C).requires_grad_()
    g1, g2 = rn(B, T, C), rn(B, T, C)
    g12 = (g1.float() + g2.float()).to(torch.bfloat16)
    y = F.pretrain_tmix_lnx_rkvres_xg_bf16(x, r, k, v, r_k, weight, bias, g)
    assert torch.isfinite(y.float()).all()

    def grads(go):
        return [t.float() for t in torch.autograd.grad(y, [x, r, r_k, weight, bias], go, retain_graph=True)]

    a, b, c = grads(g1), grads(g2), grads(g12)
    for p, q, s, name in zip(a, b, c, ("d x", "d r", "d r_k", "d weight", "d bias")):
        assert rel_rmse((p + q).cpu(), s.cpu()) <= 1.5e-2, name
