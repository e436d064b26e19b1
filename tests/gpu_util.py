"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

DEV = "cuda:0"

# Tolerance of the dense paths: normalised max error against the reference's fp32 CPU result.
# The tensor-core kernels accumulate hi*hi + lo*hi + hi*lo (3xTF32) in fp32; the summation order
# differs from the CPU's sequential sum, so agreement is to rounding, not bit for bit.
REL_TOL = 1e-4


def to_dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV)


def rel_err(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    if want.size == 0:
        return 0.0
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def pair(v):
    return [v, v] if np.isscalar(v) else list(v)


def kaiming(rng, shape):
    fan_in = int(np.prod(shape[1:]))
    return (rng.standard_normal(shape) * np.sqrt(2.0 / max(fan_in, 1))).astype(np.float32)
