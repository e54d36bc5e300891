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
