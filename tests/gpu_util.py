"""Helpers for the GPU parity tests: numpy <-> device buffers (torch is plumbing only)."""
from __future__ import annotations

import numpy as np
import torch


class Dev:
    """A device buffer made from a numpy array; ``ptr`` is what the C-ABI receives."""

    def __init__(self, arr: np.ndarray):
        arr = np.ascontiguousarray(arr)
        self.dtype = arr.dtype
        self.shape = arr.shape
        self.t = torch.from_numpy(arr.view(np.uint8).reshape(-1).copy()).cuda()

    @property
    def ptr(self) -> int:
        return self.t.data_ptr()

    def get(self) -> np.ndarray:
        torch.cuda.synchronize()
        return self.t.cpu().numpy().view(self.dtype).reshape(self.shape)


def zeros(shape, dtype) -> Dev:
    return Dev(np.zeros(shape, dtype))


def f32(v: float) -> Dev:
    return Dev(np.array([v], np.float32))


def rand_bf16(rng: np.random.Generator, shape, scale=1.0) -> np.ndarray:
    """bf16 bit patterns (uint16) of N(0, scale^2) samples."""
    from oracle import oracle as O
    return O.f32_to_bf16_bits((rng.standard_normal(shape) * scale).astype(np.float32))


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))
