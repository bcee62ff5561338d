"""Input generators shared by the CPU and GPU tests.

Two families: the closed-form generators of the reference's own device tests
(restated so the same cases can be run here), and seeded synthetic tensors with
the shapes and value distributions of the benchmark configurations.
"""
from __future__ import annotations

import numpy as np


def lcg_bytes(n: int, seed: int) -> np.ndarray:
    """The byte LCG of the reference's integer tests
    (crates/onnx-vulkan-core/tests/matmul_integer_variants.rs:29-37)."""
    state = (seed | 1) & 0xFFFFFFFFFFFFFFFF
    out = np.empty(n, dtype=np.uint8)
    for i in range(n):
        state = (state * 6364136223846793005 + 1) & 0xFFFFFFFFFFFFFFFF
        out[i] = (state >> 33) & 0xFF
    return out


def lcg_bytes_fast(n: int, seed: int) -> np.ndarray:
    """Same sequence as lcg_bytes, vectorised in blocks (for large n)."""
    if n <= 4096:
        return lcg_bytes(n, seed)
    a, c, mask = 6364136223846793005, 1, (1 << 64) - 1
    block = 4096
    # per-offset affine maps x -> A_j x + C_j for j = 1..block
    A = np.empty(block, dtype=object)
    Cc = np.empty(block, dtype=object)
    aj, cj = 1, 0
    for j in range(block):
        aj, cj = (aj * a) & mask, (cj * a + c) & mask
        A[j], Cc[j] = aj, cj
    A64 = np.array([int(v) for v in A], dtype=np.uint64)
    C64 = np.array([int(v) for v in Cc], dtype=np.uint64)
    out = np.empty(n, dtype=np.uint8)
    state = np.uint64((seed | 1) & mask)
    pos = 0
    with np.errstate(over="ignore"):
        while pos < n:
            m = min(block, n - pos)
            states = A64[:m] * state + C64[:m]
            out[pos:pos + m] = (states >> np.uint64(33)).astype(np.uint8)
            state = states[m - 1]
            pos += m
    return out


# (M, K, N, block_size): crates/onnx-vulkan-core/tests/matmul_nbits.rs:167-252
NBITS_REFERENCE_CASES = [
    (1, 1152, 256, 32),
    (5, 256, 48, 32),
    (2, 100, 17, 32),
    (1, 128, 4096, 32),
    (1, 96, 65536, 32),
    (3, 128, 4096, 32),
    (1, 80, 33, 16),
]


def nbits_reference_case(m, k, n, block_size):
    """Closed-form inputs of tests/matmul_nbits.rs:64-78: nibble ramp
    (7 col + 3 k) % 16, zero point (col + 5 b) % 16, scale ((3 col + b) % 11)/32
    - 0.15, a[i] = ((13 i) % 29 - 14)/8.  Returns unpacked arrays."""
    nb = -(-k // block_size)
    col = np.arange(n)[:, None]
    kk = np.arange(k)[None, :]
    nib = ((col * 7 + kk * 3) % 16).astype(np.uint8)
    b = np.arange(nb)[None, :]
    zp = ((col + b * 5) % 16).astype(np.uint8)
    scale = (((col * 3 + b) % 11).astype(np.float32) / np.float32(32.0) - np.float32(0.15))
    a = ((np.arange(m * k) * 13 % 29).astype(np.float32) - np.float32(14.0)) / np.float32(8.0)
    return a.reshape(m, k), nib, zp, scale.astype(np.float32)


def nbits_expected_f64(a, nib, zp, scale, block_size):
    """The scalar reference of tests/matmul_nbits.rs:79-91 in float64."""
    k = nib.shape[1]
    blk = np.arange(k) // block_size
    w = (nib.astype(np.float64) - zp[:, blk].astype(np.float64)) * scale[:, blk].astype(np.float64)
    return a.astype(np.float64) @ w.T


def rng_for(config: int, tensor: int) -> np.random.Generator:
    """One PCG64 stream per (benchmark configuration, tensor index)."""
    return np.random.Generator(np.random.PCG64(0xB2000000 + 0x100 * config + tensor))


def nbits_synthetic(config, m, k, n, block_size, real=np.float16, scale_lo=0.002, scale_hi=0.02,
                    with_zp=True):
    """Seeded int4 weights with the distributions of the benchmark configs:
    activations N(0,1), nibbles and zero points uniform 0..15, scales uniform."""
    nb = -(-k // block_size)
    a = rng_for(config, 0).standard_normal((m, k), dtype=np.float32).astype(real)
    nib = rng_for(config, 1).integers(0, 16, size=(n, k), dtype=np.uint8)
    scale = rng_for(config, 2).uniform(scale_lo, scale_hi, size=(n, nb)).astype(np.float32).astype(real)
    zp = rng_for(config, 3).integers(0, 16, size=(n, nb), dtype=np.uint8) if with_zp else None
    return a, nib, zp, scale


def xorshift_dql_input(count: int = 1 << 20) -> np.ndarray:
    """crates/onnx-vulkan-core/tests/dynamic_quantize.rs:90-102."""
    mask = (1 << 64) - 1
    state = 0x9E3779B97F4A7C15
    out = np.empty(count, dtype=np.float32)
    for i in range(count):
        state ^= (state << 13) & mask
        state ^= state >> 7
        state ^= (state << 17) & mask
        out[i] = np.float32(np.float32(state >> 40) / np.float32(1 << 24)) * np.float32(5.3) - np.float32(1.9)
    return out


def dql_ramp(r: float, n: int = 2048) -> np.ndarray:
    """crates/onnx-vulkan-core/tests/dynamic_quantize.rs:78-87, in f32 steps."""
    r = np.float32(r)
    i = np.arange(n, dtype=np.float32)
    return (-r + np.float32(2.0) * r * i / np.float32(n - 1)).astype(np.float32)


def dql_numpy(x: np.ndarray):
    """DynamicQuantizeLinear by its definition in numpy float32 (IEEE divide,
    ties to even), independent of the C oracle."""
    x = x.astype(np.float32).reshape(-1)
    mn = np.float32(min(0.0, float(x.min()))) if x.size else np.float32(0)
    mx = np.float32(max(0.0, float(x.max()))) if x.size else np.float32(0)
    scale = np.float32(1.0) if mx == mn else np.float32((mx - mn) / np.float32(255.0))
    zp = np.rint(np.clip(np.float32(-mn / scale), 0, 255)).astype(np.float32)
    y = np.clip(np.rint((x / scale).astype(np.float32)) + zp, 0, 255).astype(np.uint8)
    return y, scale, int(zp)
