"""In-tree build of the native code (run `python -m flashrwkv_b200.build`).

Two artefacts land inside the package directory:

* ``libfrwkv_b200.so`` -- every CUDA kernel plus the C ABI of
  ``include/frwkv_b200.h``, compiled by nvcc for sm_100a only.  No Torch types.
* ``_C*.so`` -- the PyTorch C++ host layer (``csrc/torch_binding.cpp``), compiled
  by g++ against the Torch headers and linked to the library above.

nvcc cross-compiles without a GPU, so the build works on a CPU-only machine.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
LIB = PKG / "libfrwkv_b200.so"

CUDA_SOURCES = [
    "frwkv_capi.cu",
    "metadata.cu",
    "wkv7_recurrent.cu",
    "wkv7_recurrent_fp16.cu",
    "wkv7_recurrent_wide.cu",
    "wkv7_chunk_fwd.cu",
    "wkv7_chunk_fused.cu",
    "wkv7_chunk_bwd.cu", "wkv7_checkpoints.cu", "wkv7_train_wide.cu", "tmix_decode_layer.cu",
    "tmix_elementwise.cu",
    "tmix_norm.cu",
    "tmix_train.cu",
    "tmix_linear.cu",
    "tmix_gemm_tma.cu",
    "wkv7_backward.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    *os.environ.get("FRWKV_EXTRA_NVCC_FLAGS", "").split(),
]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else (shutil.which("nvcc") or "nvcc")


def _host_cxx() -> str:
    # the system compiler; an inherited CXX may point at a toolchain without its runtime specs
    return shutil.which("g++") or "g++"


def _digest(paths, extra=()) -> str:
    h = hashlib.sha256()
    for p in sorted(str(x) for x in paths):
        h.update(Path(p).name.encode())
        h.update(Path(p).read_bytes())
    for e in extra:
        h.update(str(e).encode())
    return h.hexdigest()


def _up_to_date(target: Path, digest: str) -> bool:
    """A built file is current when its stamp (a hash of its sources and flags) matches; file times
    are not used because copies of the tree do not always keep them."""
    stamp = target.with_suffix(target.suffix + ".stamp")
    return target.exists() and stamp.exists() and stamp.read_text().strip() == digest


def _write_stamp(target: Path, digest: str) -> None:
    target.with_suffix(target.suffix + ".stamp").write_text(digest + "\n")


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    proc = subprocess.run([str(c) for c in cmd], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError(f"build step failed: {cmd[0]} (exit {proc.returncode})")
    if verbose and proc.stdout.strip():
        print(proc.stdout)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile the kernels and the C ABI into libfrwkv_b200.so (one nvcc call per source, then link)."""
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    lib_digest = _digest([CSRC / n for n in CUDA_SOURCES] + headers, NVCC_FLAGS)
    if not force and not ptxas_info and _up_to_date(LIB, lib_digest):
        return LIB
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    objs = []
    for name in CUDA_SOURCES:
        src = CSRC / name
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        obj_digest = _digest([src] + headers, NVCC_FLAGS)
        if not force and not ptxas_info and _up_to_date(obj, obj_digest):
            continue
        flags = list(NVCC_FLAGS)
        if ptxas_info:
            flags += ["-Xptxas", "-v"]
        _run([_nvcc(), *flags, "-ccbin", _host_cxx(), f"-I{INCLUDE}", f"-I{CSRC}", "-c", src, "-o", obj],
             verbose or ptxas_info)
        _write_stamp(obj, obj_digest)
    _run([_nvcc(), "-shared", "-ccbin", _host_cxx(), "-o", LIB, *objs], verbose)
    _write_stamp(LIB, lib_digest)
    return LIB


def torch_ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / f"_C{suffix}"


def build_torch_ext(force: bool = False, verbose: bool = False) -> Path:
    """Compile csrc/torch_binding.cpp into the `_C` extension module, linked to libfrwkv_b200.so."""
    import torch
    from torch.utils import cpp_extension

    out = torch_ext_path()
    src = CSRC / "torch_binding.cpp"
    digest = _digest([src, *INCLUDE.glob("*.h")], [torch.__version__])
    if not force and _up_to_date(out, digest):
        return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    includes = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], f"{cuda_home}/include",
                str(INCLUDE)]
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [_host_cxx(), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-DUSE_CUDA", "-Wno-deprecated-declarations",
           *[f"-I{p}" for p in includes], str(src), "-o", str(out),
           f"-L{PKG}", "-lfrwkv_b200", f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
           "-ltorch", "-ltorch_python", f"-L{cuda_home}/lib64", "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    _write_stamp(out, digest)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_torch_ext(force=force, verbose=verbose)


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers/spills per kernel")
    ns = ap.parse_args()
    build_library(force=ns.force, verbose=ns.verbose, ptxas_info=ns.ptxas_info)
    build_torch_ext(force=ns.force, verbose=ns.verbose)
    print("built", LIB.name, "and", torch_ext_path().name)
