"""Shared scenario builders for the parity tests: seeded inputs that go, bit for bit, both to
the CPU checker (oracle/) and to the CUDA path."""
from __future__ import annotations

import numpy as np

from oracle import cbind as ob


def randn_bits(rng: np.random.Generator, shape, dtype: int) -> np.ndarray:
    """N(0,1) samples rounded to the storage type, as uint16 bit patterns."""
    return ob.from_float(rng.standard_normal(shape, dtype=np.float32), dtype)


def shuffled_free_stack(engine, rng: np.random.Generator) -> None:
    """Leaves the pool's free stack in a seeded random order using only the public pool calls:
    take every page, then give them back in a shuffled order."""
    n = engine.max_blocks()
    pages = [engine.alloc_block() for _ in range(n)]
    assert sorted(pages) == list(range(n))
    for p in rng.permutation(n):
        engine.free_block(int(p))


def ulp(x: np.ndarray, dtype: int) -> np.ndarray:
    """Spacing of the storage type at |x| (fp16: 10 mantissa bits, bf16: 7)."""
    bits = 10 if dtype == ob.F16 else 7
    a = np.maximum(np.abs(x.astype(np.float64)), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(a)) - bits)


def torch_bits(t):
    """uint16 view of a 2-byte torch tensor as numpy."""
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def to_dev(bits: np.ndarray, dtype: int, device="cuda"):
    import torch
    t = torch.from_numpy(bits.view(np.int16)).to(device)
    return t.view(torch.float16 if dtype == ob.F16 else torch.bfloat16)


def rope_fastmath_tolerance(x_bits, rot, theta, pos, dtype):
    """Largest difference to expect, per element of rows [..., D], between an accurately evaluated RoPE and
    the reference's device code built with --use_fast_math: __sinf/__cosf are off by about 2^-21.4 * |angle|
    (CUDA programming guide, intrinsic error table) and __powf's relative error carries into the angle, so
    the rotated value may move by (|x0| + |x1|) * angle * 2e-6 in addition to one rounding of the result."""
    x = ob.to_float(x_bits, dtype).astype(np.float64)
    half = rot // 2
    angle = pos / theta ** (2.0 * np.arange(half) / rot)
    mag = np.abs(x[..., :half]) + np.abs(x[..., half:rot])
    tol = np.zeros_like(x)
    tol[..., :half] = mag * (angle * 2e-6 + 2e-6)
    tol[..., half:rot] = tol[..., :half]
    return tol
