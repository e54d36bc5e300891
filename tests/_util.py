"""Helpers shared by the tests: golden-vector loading and error metrics."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"

# io dtype of the 16-bit arrays (stored as uint16 bit patterns) in each golden file
_IO_DTYPE = {
    "recurrent_ragged": torch.bfloat16,
    "recurrent_fp16state": torch.float16,
    "recurrent_fp16state_d128": torch.float16,
    "chunk_bf16": torch.bfloat16,
    "rl_fp16": torch.float16,
    "statetune": torch.float16,
    "pretrain": torch.bfloat16,
    "tmix_kk_a_gate": torch.float16,
    "tmix_lnx": torch.float16,
    "tmix_vres": torch.float16,
    "tmix_mix6": torch.float16,
    "tmix_lowrank": torch.float16,
    "tmix_norm": torch.float16,
}


def load_golden(name: str) -> dict:
    """Load tests/golden/<name>.npz as torch tensors (16-bit arrays keep their dtype)."""
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as z:
        for key in z.files:
            arr = z[key]
            if arr.dtype == np.uint16:
                out[key] = torch.from_numpy(arr.view(np.int16).copy()).view(_IO_DTYPE[name])
            elif arr.ndim == 0:
                out[key] = float(arr)
            else:
                out[key] = torch.from_numpy(arr.copy())
    return out


def rel_rmse(actual, expected) -> float:
    """The reference's tolerance metric: ||a-e||_rms / ||e||_rms."""
    a = torch.as_tensor(np.asarray(actual) if not isinstance(actual, torch.Tensor) else actual).double()
    e = torch.as_tensor(np.asarray(expected) if not isinstance(expected, torch.Tensor) else expected).double()
    denom = e.square().mean().sqrt().clamp_min(1e-30)
    return float((a - e).square().mean().sqrt() / denom)


def max_abs(actual, expected) -> float:
    a = torch.as_tensor(np.asarray(actual) if not isinstance(actual, torch.Tensor) else actual).double()
    e = torch.as_tensor(np.asarray(expected) if not isinstance(expected, torch.Tensor) else expected).double()
    return float((a - e).abs().max())
