"""The C-ABI library loads and exports every function include/*.h declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions():
    names = []
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names += re.findall(r"\b(frwkv_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_entry_points():
    names = _declared_functions()
    assert "frwkv_wkv7_recurrent_fp32io16_forward_varlen" in names
    assert "frwkv_validate_recurrent_metadata" in names


def test_library_exports_every_declared_symbol():
    from flashrwkv_b200 import _ext

    lib = _ext.capi()
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert lib.frwkv_abi_version() >= 1
    assert lib.frwkv_last_error() == b""


def test_argument_errors_are_reported_without_a_device():
    """Null pointers and bad sizes are rejected before any CUDA call."""
    from flashrwkv_b200 import _ext

    lib = _ext.capi()
    rc = lib.frwkv_validate_recurrent_metadata(None, None, 1, 1, 1, None, None, None, None)
    assert rc == -1 and b"null pointer" in lib.frwkv_last_error()
    one = ctypes.c_void_p(16)
    rc = lib.frwkv_validate_recurrent_metadata(one, one, 70000, 1, 1, one, one, one, None)
    assert rc == -1 and b"65535" in lib.frwkv_last_error()


def test_misaligned_pointers_are_rejected_without_a_device():
    """The chunk kernels move rows as 16- and 32-byte vectors; a pointer that is not 32-byte aligned is an argument
    error, reported before any CUDA call, and not a fault on the device."""
    from flashrwkv_b200 import _ext

    lib = _ext.capi()
    ok, bad = ctypes.c_void_p(4096), ctypes.c_void_p(4096 + 8)
    f = ctypes.c_float(1.0)
    # frwkv_wkv7_chunk_backward(sco, cs, ce, final_state, boundary, adjoint, sda, r, w, k, v, a, b, bias, dy,
    #                           dr, dw, dk, dv, da, db, error_flag, status, T, B, Cn, H, D, dtype, scale, stream)
    args = [ok] * 3 + [ok] * 4 + [ok] * 6 + [None, ok] + [ok] * 6 + [None, None, 64, 1, 1, 1, 64, 1, f, None]
    args[9] = bad  # k
    assert lib.frwkv_wkv7_chunk_backward(*args) == -1
    assert b"32-byte aligned" in lib.frwkv_last_error()
    # frwkv_wkv7_chunk_fused_fp32io16_forward(sco, cs, ce, state_indices, status, pool, r, w, k, v, a, b, bias,
    #                                         y, y32, boundary, sda, error_flag, T, B, Cn, H, D, dtype, scale, stream)
    args = [ok] * 3 + [None, None, ok] + [ok] * 6 + [None, bad, None, None, None, None, 64, 1, 1, 1, 64, 1, f, None]
    assert lib.frwkv_wkv7_chunk_fused_fp32io16_forward(*args) == -1
    assert b"32-byte aligned" in lib.frwkv_last_error()


def test_python_surface_matches_reference_signatures():
    import inspect

    import flashrwkv_b200 as F

    sig = inspect.signature(F.infer_recurrent_fp32io16_forward_varlen)
    names = list(sig.parameters)
    assert names[:6] == ["r", "decay_logits", "k", "v", "a", "b"]
    for kwonly in ("state_pool", "cu_seqlens", "state_indices", "scale", "decay_bias", "max_seqlen",
                   "validated_metadata"):
        assert sig.parameters[kwonly].kind is inspect.Parameter.KEYWORD_ONLY
    assert "log_decay" not in names
    sig = inspect.signature(F.prepare_recurrent_metadata)
    assert list(sig.parameters) == ["cu_seqlens", "state_indices", "total_tokens", "state_pool_size", "max_seqlen"]


def test_host_validation_runs_before_any_launch():
    import torch

    import flashrwkv_b200 as F

    t = torch.zeros(4, 2, 64, dtype=torch.bfloat16)
    pool = torch.zeros(2, 2, 64, 64)
    cu = torch.tensor([0, 4], dtype=torch.int32)
    idx = torch.tensor([0], dtype=torch.int32)
    with pytest.raises(TypeError, match="r must be a torch.Tensor"):
        F.infer_recurrent_fp32io16_forward_varlen(object(), t, t, t, t, t, state_pool=pool, cu_seqlens=cu,
                                                  state_indices=idx)
    with pytest.raises(ValueError, match=r"packed shape \[total_tokens,H,D\]"):
        F.infer_recurrent_fp32io16_forward_varlen(t.reshape(-1, 64), t, t, t, t, t, state_pool=pool, cu_seqlens=cu,
                                                  state_indices=idx)
    with pytest.raises(TypeError, match="float32"):
        F.infer_recurrent_fp32io16_forward_varlen(t, t, t, t, t, t, state_pool=pool.half(), cu_seqlens=cu,
                                                  state_indices=idx)
    with pytest.raises(TypeError, match="cu_seqlens must be a torch.Tensor"):
        F.infer_recurrent_fp32io16_forward_varlen(t, t, t, t, t, t, state_pool=pool, cu_seqlens=[0, 4],
                                                  state_indices=idx)
    # CPU tensors reach the native check and are refused there (no fallback)
    with pytest.raises((ValueError, RuntimeError), match="CUDA"):
        F.infer_recurrent_fp32io16_forward_varlen(t, t, t, t, t, t, state_pool=pool, cu_seqlens=cu,
                                                  state_indices=idx)
