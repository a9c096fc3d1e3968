"""Shared helpers of the test-suite: seeded inputs, dtype plumbing, error metrics."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as O

CODES = {"float32": O.F32, "float16": O.F16, "bfloat16": O.BF16}
TORCH = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}

# element counts around every boundary of the kernels (vector width 4, pass 1024,
# chunk 4096, the reference's chunk 65536) plus empty and one large ragged case
EDGE_NUMELS = [0, 1, 3, 4, 5, 31, 32, 33, 1023, 1024, 1025, 4095, 4096, 4097, 8191, 65535, 65536,
               65537, (1 << 20) + 3]


def make_grad(rng, n, dtype, std=1e-3, loss_scale=1.0):
    """Gradient ~N(0, std) * loss_scale in ``dtype``; numpy array (bf16 as uint16 bits)."""
    g = (rng.standard_normal(n) * std * loss_scale).astype(np.float32)
    return O.cast(g, CODES[dtype]) if dtype != "float32" else g


def to_torch(a: np.ndarray, dtype: str, device="cuda") -> torch.Tensor:
    if dtype == "bfloat16":
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(a.copy()).to(device)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max |a-b| / (|b| + rms(b)): relative error that does not blow up on the few
    elements that sit next to zero."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    if a.size == 0:
        return 0.0
    rms = float(np.sqrt(np.mean(b * b)))
    den = np.abs(b) + (rms if rms > 0 else 1e-30)
    return float(np.max(np.abs(a - b) / den))


def bits_equal(a: np.ndarray, b: np.ndarray) -> bool:
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    return a.tobytes() == b.tobytes()
