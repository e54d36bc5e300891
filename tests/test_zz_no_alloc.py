"""The allocation-free chunked forward (built-in workspace) against the ordinary entry point.

Hosts that have handed all device memory to fixed pools, or that run where an allocation could stall the device,
call `frwkv_wkv7_chunk_fp32io16_forward_noalloc`; it must give what `frwkv_wkv7_chunk_fp32io16_forward` gives with
a caller-provided workspace.  Both are called here through the C ABI with raw device pointers, twice in a row (the
second call finds the previous call's tiles in the shared array), and sizes beyond the built-in limit must be
refused.  This file sorts last on purpose, and passes on its own in a fresh process as well.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _call(lib, fn_name, meta, pool, toks, y, y32, workspace, N, B, Cn, H, scale):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    sco, cs, ce = meta
    head = [_p(sco), _p(cs), _p(ce), None, None, _p(pool), *(_p(t) for t in toks), None, _p(y), _p(y32), None]
    tail = [_p(flag), N, B, Cn, H, 64, 1, ctypes.c_float(scale), stream]
    fn = getattr(lib, fn_name)
    if workspace is not None:
        rc = fn(*head, _p(workspace), ctypes.c_size_t(workspace.numel()), *tail)
    else:
        rc = fn(*head, *tail)
    return rc, flag


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row(oracle):
    from flashrwkv_b200 import _ext, synthetic
    from flashrwkv_b200.tmix.wkv7 import make_chunk_metadata

    lib = _ext.capi()
    lib.frwkv_wkv7_chunk_workspace_bytes.restype = ctypes.c_size_t
    lib.frwkv_wkv7_chunk_noalloc_max_items.restype = ctypes.c_size_t
    assert lib.frwkv_wkv7_chunk_noalloc_max_items() == 256
    H, D = 8, 64
    lengths = (130, 64, 17, 200)               # 3 + 1 + 1 + 4 = 9 chunks x 8 heads = 72 (chunk, head) pairs
    N, B = sum(lengths), len(lengths)
    cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device="cuda")
    meta = make_chunk_metadata(cu, 64)
    Cn = meta[1].numel()
    for call in range(2):
        toks = [t.cuda() for t in synthetic.wkv7_inputs(N, H, D, seed=40 + call)]
        pool0 = synthetic.state_pool(B, H, D, seed=50 + call, device="cuda")
        ws = torch.empty(lib.frwkv_wkv7_chunk_workspace_bytes(Cn, H), dtype=torch.uint8, device="cuda")
        pool_a, pool_b = pool0.clone(), pool0.clone()
        y_a, y_b = torch.empty_like(toks[3]), torch.empty_like(toks[3])
        y32_a, y32_b = (torch.empty(N, H, D, device="cuda") for _ in range(2))
        rc, flag = _call(lib, "frwkv_wkv7_chunk_fp32io16_forward", meta, pool_a, toks, y_a, y32_a, ws, N, B, Cn, H, 0.9)
        assert rc == 0, lib.frwkv_last_error()
        rc, flag_b = _call(lib, "frwkv_wkv7_chunk_fp32io16_forward_noalloc", meta, pool_b, toks, y_b, y32_b, None, N, B,
                           Cn, H, 0.9)
        assert rc == 0, lib.frwkv_last_error()
        torch.cuda.synchronize()
        assert int(flag.item()) == 0 and int(flag_b.item()) == 0
        # same kernels, same inputs: the tolerance of the chunk tests (2e-2 max-abs on the fp32 output, 1e-3
        # relative on the state) is met with room to spare - the results are in fact identical
        assert float((y32_a - y32_b).abs().max()) <= 2e-2
        assert float((pool_a - pool_b).norm() / pool_a.norm()) <= 1e-3
        assert torch.equal(y_a, y_b) and torch.equal(pool_a, pool_b)
        assert not torch.equal(pool_a, pool0)
        # and against the CPU oracle on the same 16-bit inputs, with the parity bars of the chunk tests
        want = oracle.forward(*(t.cpu() for t in toks), state_pool=pool0.cpu(), cu_seqlens=cu.cpu(), scale=0.9)
        assert float((y32_b.cpu() - torch.from_numpy(want["y"])).abs().max()) <= 2e-2
        ref_pool = torch.from_numpy(want["state_pool"])
        assert float((pool_b.cpu() - ref_pool).norm() / ref_pool.norm()) <= 1e-3


def test_noalloc_entry_refuses_sizes_beyond_its_workspace():
    from flashrwkv_b200 import _ext

    lib = _ext.capi()
    one = ctypes.c_void_p(256)
    rc = lib.frwkv_wkv7_chunk_fp32io16_forward_noalloc(one, one, one, None, None, one, one, one, one, one, one, one, None,
                                                       one, None, None, None, 64 * 9, 1, 9, 32, 64, 1, ctypes.c_float(1.0),
                                                       None)
    assert rc == -1
    assert b"exceeds the built-in workspace" in lib.frwkv_last_error()
