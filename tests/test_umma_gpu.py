"""Pins the tcgen05 descriptor encodings: one tensor-core product per tile shape and chunk stride vs numpy."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tf32(x: np.ndarray) -> np.ndarray:
    bits = x.astype(np.float32).view(np.uint32)
    bits = ((bits + 0x1000) & 0xFFFFE000).astype(np.uint32)
    return bits.view(np.float32)


CASES = [
    # n, a_stride, b_stride     (the tile shapes used by the chunk kernels)
    (128, 2048, 2048),   # [A~;R~] x [B~;K~]^T
    (64, 2048, 1040),    # [A_ak;-] x V ; scan: [E;M] x S
    (64, 2064, 1040),    # [A~^T;Z^T] x T^T ; [A_rk;K^^T] x V
    (128, 2064, 2048),   # [A_rb;B^^T] x [P|Q]
]


@pytest.mark.parametrize("n,a_stride,b_stride", CASES)
def test_single_mma_matches_numpy(n, a_stride, b_stride):
    from flashrwkv_b200 import _ext

    lib = _ext.capi()
    rng = np.random.default_rng(n + a_stride + b_stride)
    A = rng.standard_normal((128, 64)).astype(np.float32)
    Bm = rng.standard_normal((n, 64)).astype(np.float32)
    a_d, b_d = torch.from_numpy(A).cuda(), torch.from_numpy(Bm).cuda()
    d_d = torch.zeros(128, n, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.frwkv_selftest_umma(p(a_d), p(b_d), p(d_d), n, a_stride, b_stride, -1, p(flag),
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.frwkv_last_error()
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "the MMA never signalled completion"
    want = _tf32(A).astype(np.float64) @ _tf32(Bm).astype(np.float64).T
    got = d_d.cpu().numpy()
    assert np.abs(got - want).max() < 2e-4, np.abs(got - want).max()
