"""Pins the tcgen05 descriptor encodings: one tensor-core product per operand orientation vs numpy."""
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
    # n, a_mn, b_mn, a_stride, b_stride     (the forms used by the chunk kernels)
    (128, 0, 0, 2048, 2048),   # [B~;K~] x [A~;R~]^T
    (64, 1, 1, 1024, 2048),    # [A_ak;A_rk] x V  (V interleaved with another tile)
    (64, 1, 1, 2048, 1024),    # [A~|Z]^T x T^T
    (128, 1, 0, 1024, 2048),   # [A_rb;B^] x [P|Q]
    (64, 0, 1, 2048, 1024),    # scan: [E;M] x S
]


@pytest.mark.parametrize("n,a_mn,b_mn,a_stride,b_stride", CASES)
def test_single_mma_matches_numpy(n, a_mn, b_mn, a_stride, b_stride):
    from flashrwkv_b200 import _ext

    lib = _ext.capi()
    rng = np.random.default_rng(n + 2 * a_mn + b_mn)
    A = rng.standard_normal((128, 64)).astype(np.float32)
    Bm = rng.standard_normal((n, 64)).astype(np.float32)
    a_d, b_d = torch.from_numpy(A).cuda(), torch.from_numpy(Bm).cuda()
    d_d = torch.zeros(128, n, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.frwkv_selftest_umma(p(a_d), p(b_d), p(d_d), n, a_mn, b_mn, a_stride, b_stride, -1, p(flag),
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.frwkv_last_error()
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "the MMA never signalled completion"
    want = _tf32(A).astype(np.float64) @ _tf32(Bm).astype(np.float64).T
    got = d_d.cpu().numpy()
    assert np.abs(got - want).max() < 2e-4, np.abs(got - want).max()
