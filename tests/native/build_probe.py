"""Builds tests/native/libfrwkv_probe.so: test-only kernels (tensor-core probes, a bounded wait that runs out).

Kept apart from the product library on purpose: nothing under flashrwkv_b200/ links or loads it.
Run `python -m tests.native.build_probe`, or let tests/conftest.py do it at session start.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

from flashrwkv_b200 import build as native

HERE = Path(__file__).resolve().parent
SOURCES = [HERE / "umma_probe.cu"]
LIB = HERE / "libfrwkv_probe.so"


def build(force: bool = False, verbose: bool = False) -> Path:
    headers = list(native.CSRC.glob("*.cuh"))
    digest = native._digest(SOURCES + headers, native.NVCC_FLAGS)
    if not force and native._up_to_date(LIB, digest):
        return LIB
    native._run([native._nvcc(), *native.NVCC_FLAGS, "-ccbin", native._host_cxx(), f"-I{native.CSRC}",
                 f"-I{native.INCLUDE}", "-shared", *SOURCES, "-o", LIB], verbose)
    native._write_stamp(LIB, digest)
    return LIB


def load() -> ctypes.CDLL:
    return ctypes.CDLL(str(build()))


if __name__ == "__main__":
    print(build(force=True, verbose=True))
