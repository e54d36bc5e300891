"""Loader of the native code.  There is no fallback: a missing build raises."""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libfrwkv_b200.so"
_C = None
_capi = None


class ExtensionNotBuilt(RuntimeError):
    pass


def extension():
    """The `_C` PyTorch extension module (host layer over the C ABI)."""
    global _C
    if _C is None:
        try:
            import torch  # noqa: F401  (libtorch must be loaded before the extension)
            from . import _C as module
        except ImportError as exc:
            raise ExtensionNotBuilt(
                "flashrwkv_b200 native extension is not built; run `python -m flashrwkv_b200.build` "
                f"(there is no CPU or PyTorch fallback): {exc}"
            ) from exc
        _C = module
    return _C


def capi() -> ctypes.CDLL:
    """libfrwkv_b200.so opened through ctypes (the raw C ABI of include/frwkv_b200.h)."""
    global _capi
    if _capi is None:
        if not _LIB_PATH.exists():
            raise ExtensionNotBuilt(
                f"{_LIB_PATH.name} is not built; run `python -m flashrwkv_b200.build`")
        lib = ctypes.CDLL(str(_LIB_PATH))
        lib.frwkv_last_error.restype = ctypes.c_char_p
        lib.frwkv_abi_version.restype = ctypes.c_int
        _capi = lib
    return _capi


def library_path() -> Path:
    return _LIB_PATH


def device_error_flags() -> dict:
    """The device error words of the latest launches that use bounded waits, by stage name (a host read: this
    synchronises).  Non-zero = a tensor-core, copy or grid-barrier wait ran out in that stage and its outputs are NaN.
    Stages: `wkv7_chunk_forward`, `wkv7_chunk_backward`, `tmix_linear` (sticky, one word per device),
    `tmix_decode_layer` (word 7 of its eight); the recurrent decode kernels report through the metadata status word
    (bit 16) instead."""
    out = {}
    for stage, words in extension().last_error_flags().items():
        out[stage] = int(words[7].item()) if stage == "tmix_decode_layer" else int(words.flatten()[0].item())
    return out


def check_device_error_flags() -> None:
    """Raise `RuntimeError` if any stage of `device_error_flags()` reports a wait that ran out."""
    bad = {stage: flag for stage, flag in device_error_flags().items() if flag != 0}
    if bad:
        raise RuntimeError(f"a bounded device wait ran out (stage -> error word): {bad}; the affected outputs are NaN")
