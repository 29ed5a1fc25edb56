"""CPU: the library's host-side constructors (limits, RoPE tables) against the
reference fixtures and the oracle.  Integer results are bit-exact."""
import json
import os

import numpy as np
import pytest

import oracle_lib as O
from qwen_metal_b200 import abi, workloads

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel_l2(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-30)))


def test_prefix_limits_bit_exact():
    layouts = [
        [(20, 0), (48, 1), (17, 0), (64, 1)],
        [(64, 0), (256, 1)],
        [(256, 0), (4096, 1), (4096, 1)],
        [(1, 0), (1, 1)],
        [(0, 0), (5, 1), (0, 1), (3, 0)],
    ]
    for runs in layouts:
        assert np.array_equal(abi.prefix_limits(runs), O.prefix_limits(runs))


def test_rope_tables_match_reference_fixtures():
    t = np.load(os.path.join(GOLD, "ref_rope_tables.npz"))
    for grid in (4, 8):
        cos, sin = abi.rope_tables(23, grid, grid)
        assert rel_l2(cos, t[f"pipeline_cos_{grid}"]) <= 1e-6
        assert rel_l2(sin, t[f"pipeline_sin_{grid}"]) <= 1e-6
    for case, bh, bw, tb in (("a", [4], [4], [0]), ("b", [3], [4], [8]),
                             ("c", [6, 8], [8, 8], [20, 17])):
        cos, sin = abi.rope_tables_blocks(bh, bw, tb)
        assert rel_l2(cos, t[f"dit_{case}_cos"]) <= 1e-6
        assert rel_l2(sin, t[f"dit_{case}_sin"]) <= 1e-6


def test_rope_tables_equal_oracle_bitwise():
    for args in ((128, 32, 32), (7, 5, 3)):
        a, b = abi.rope_tables(*args), O.rope_tables(*args)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    a = abi.rope_tables_blocks([64, 64], [64, 64], [256, 0])
    b = O.rope_tables_blocks([64, 64], [64, 64], [256, 0])
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.parametrize("index,pairs", [(1, 84000), (2, 1187904), (3, 34525332),
                                         (4, 52461696), (5, 553910784)])
def test_workload_visible_pairs(index, pairs):
    """Mask-aware work per config (text rows token-causal, key padding excluded)."""
    w = workloads.workload(index)
    assert w.visible_pairs() == pairs
    tl = np.asarray(w.text_len, np.uint32) if w.text_pad else None
    assert O.visible_pairs(w.limits(), w.batch, w.rows, w.rows, tl, w.text_pad) == pairs


def test_workload_tables_shape():
    w = workloads.workload(4)
    cos, sin = w.rope_tables()
    assert cos.shape == (8448, 64) and sin.shape == (8448, 64)
    # the second image block sits one max(gh, gw) further along the frame axis
    assert np.isclose(cos[256, 0], np.cos(256.0), atol=1e-6)
    assert np.isclose(cos[256 + 4096, 0], np.cos(256.0 + 64.0), atol=1e-6)


def test_split_tail_rule():
    """Which units of an attention launch run as two half CTAs (host arithmetic of
    the launcher): the remainder of units / SMs when doubling it still fits the SMs."""
    import ctypes as C
    lib = abi.load()
    fn = lib.qwcu_attn_sm100_tail_units
    fn.restype, fn.argtypes = C.c_uint32, [C.c_uint32, C.c_uint32]
    sms = 148
    assert fn(816, sms) == 76       # cfg3: 2 x 24 heads x 17 blocks -> 5 waves + 76
    assert fn(792, sms) == 52       # cfg4: 24 heads x 33 blocks
    assert fn(3168, sms) == 60      # cfg5
    assert fn(102, sms) == 0        # cfg3 on one of eight GPUs: 204 halves would not fit
    assert fn(204, sms) == 56       # ... on one of four
    assert fn(148 * 7, sms) == 0    # full waves only
    assert fn(48, sms) == 48        # fewer units than SMs: every unit is split
    assert fn(10, 0) == 0
    for units in range(1, 2000):
        tail = fn(units, sms)
        assert tail in (0, units % sms) and 2 * tail <= sms + sms // 16


def test_prefix_limits_random_layouts_and_mask_semantics():
    """Seeded random run layouts: the library's limits equal the oracle's bit for bit,
    and they mean what the reference's mask means (qwen_dit.m:1651-1665): a text row
    sees the keys up to and including itself, an image row every key up to the end of
    its own run, and limits never decrease along the joint sequence."""
    rng = np.random.default_rng(2024)
    for _ in range(200):
        runs = [(int(rng.integers(0, 40)), int(rng.integers(0, 2))) for _ in range(int(rng.integers(1, 7)))]
        if sum(r for r, _ in runs) == 0:
            continue
        got = abi.prefix_limits(runs)
        assert np.array_equal(got, O.prefix_limits(runs))
        start = 0
        for rows, is_image in runs:
            for r in range(start, start + rows):
                assert got[r] == (start + rows if is_image else r + 1)
            start += rows
        assert np.all(np.diff(got.astype(np.int64)) >= 0)
        mask = O.dense_mask(got, 1, start, start)[0]
        assert np.array_equal(mask.sum(-1), got)   # row r sees exactly the first limit[r] keys
