"""Seeded input cases for the scalar kernels of the path, shared by the golden
generator (tests/golden/make_msl_golden.py), which runs the reference's own
shader kernels on them, and by the CPU test that holds the oracle to the result.
"""
import numpy as np


def _bf16(values):
    bits = np.asarray(values, np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def head_norm_case(seed, sequence=37, heads=3):
    rng = np.random.default_rng([seed, 1])
    x = rng.standard_normal((sequence, heads, 128), dtype=np.float32)
    x[0, 0] = 0.0                      # a head of zeros: inverse = rsqrt(eps)
    x[1, 1] *= 300.0                   # large values
    x[2, 2] *= 1e-3                    # small values
    x[3, 0, 5:] = 0.0                  # one dominant element
    w = rng.standard_normal(128, dtype=np.float32) * 0.1 + 1.0
    w[7] = -0.5
    return _bf16(x), _bf16(w), sequence, heads, 1e-6


def rope_case(seed, sequence=37, heads=3):
    rng = np.random.default_rng([seed, 2])
    q = rng.standard_normal((sequence, heads, 128), dtype=np.float32) * 2.0
    k = rng.standard_normal((sequence, heads, 128), dtype=np.float32) * 2.0
    angle = rng.uniform(-50.0, 50.0, (sequence, 64))
    return (_bf16(q), _bf16(k), np.cos(angle).astype(np.float32),
            np.sin(angle).astype(np.float32), sequence, heads)


def row_case(seed, rows, width, slots=4, maps=2):
    rng = np.random.default_rng([seed, 3, width])
    x = rng.standard_normal((rows, width), dtype=np.float32) * 3.0 + 0.25
    x[0] = 1.5                          # constant row: every centred value cancels
    branch = rng.standard_normal((rows, width), dtype=np.float32)
    modulation = rng.standard_normal((maps, slots, width), dtype=np.float32) * 0.5
    row_map = (np.arange(rows) % maps).astype(np.uint32)
    return _bf16(x), _bf16(branch), _bf16(modulation), row_map, rows, width, slots


CASES = {
    "head_norm": [3, 4],
    "rope": [5],
    "rows": [(6, 9, 4096), (7, 5, 1000), (8, 3, 200)],  # (seed, rows, width)
}
