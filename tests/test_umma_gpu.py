"""Pins the tcgen05 building blocks with the test-only probe library (tests/native): descriptor encodings and
tile strides (one product per tile shape vs numpy), operands held in tensor memory, and the give-up path of the
bounded barrier wait."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tf32(x: np.ndarray) -> np.ndarray:
    bits = x.astype(np.float32).view(np.uint32)
    bits = ((bits + 0x1000) & 0xFFFFE000).astype(np.uint32)
    return bits.view(np.float32)


@pytest.fixture(scope="module")
def probe():
    from tests.native import build_probe

    return build_probe.load()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


CASES = [
    # n, a_stride, b_stride, a_in_tmem     (the tile shapes used by the chunk kernels)
    (128, 2048, 2048, 0),   # [A~;R~] x [B~;K~]^T
    (64, 2048, 1040, 0),    # [A_ak;-] x V ; scan: [E;M] x S
    (64, 2064, 1040, 0),    # [A~^T;Z^T] x T^T ; [A_rk;K^^T] x V ; [T';0] x X^T
    (128, 2064, 2048, 0),   # [A_rb;B^^T] x [P|Q]
    (128, 2048, 2048, 1),   # A in tensor memory: [A~;R~] x [B~;K~]^T
    (64, 2048, 1040, 1),    # A in tensor memory against a 64-row transposed tile
]


@pytest.mark.parametrize("n,a_stride,b_stride,a_in_tmem", CASES)
def test_single_mma_matches_numpy(probe, n, a_stride, b_stride, a_in_tmem):
    rng = np.random.default_rng(n + a_stride + b_stride + a_in_tmem)
    A = rng.standard_normal((128, 64)).astype(np.float32)
    Bm = rng.standard_normal((n, 64)).astype(np.float32)
    a_d, b_d = torch.from_numpy(A).cuda(), torch.from_numpy(Bm).cuda()
    d_d = torch.zeros(128, n, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = probe.frwkv_probe_umma(_p(a_d), _p(b_d), _p(d_d), n, a_stride, b_stride, a_in_tmem, _p(flag), _stream())
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "the MMA never signalled completion"
    want = _tf32(A).astype(np.float64) @ _tf32(Bm).astype(np.float64).T
    got = d_d.cpu().numpy()
    assert np.abs(got - want).max() < 2e-4, np.abs(got - want).max()


def test_tensor_memory_store_load_round_trip(probe):
    src = torch.randint(0, 2**30, (128, 32), dtype=torch.int32, device="cuda")
    out = torch.zeros_like(src)
    rc = probe.frwkv_probe_tmem_roundtrip(_p(src), _p(out), _stream())
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert torch.equal(out, 2 * src)


@pytest.mark.parametrize("limit", [1, 4096])
def test_bounded_wait_gives_up_and_returns(probe, limit):
    """Nothing ever arrives at the barrier: the kernel must come back with the flag set, the call with a code."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    cycles = torch.zeros(1, dtype=torch.int64, device="cuda")
    rc = probe.frwkv_probe_bounded_wait(ctypes.c_uint32(limit), _p(flag), _p(cycles), _stream())
    assert rc == -4, rc
    assert int(flag.item()) == 1
    assert int(cycles.item()) > 0
    # the context is still usable afterwards
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0
