"""The oracle's head RMSNorm (both roundings), RoPE application, AdaLN norm and
gated residual, held bit for bit to the reference's own shader kernels.

The golden file tests/golden/msl_scalar_kernels.json was produced by running the
reference's kernel text, compiled as C++ (oracle/msl_shim.h, oracle/extract_msl.py,
`make -C oracle ref`), on the seeded cases of tests/msl_cases.py.  Where that
build is present (oracle/_ref/libmsl_ref.so) the oracle is also compared with it
directly on further seeds, element by element.

Tolerance: none (bit equality).  The shim fixes the two points the Metal
language leaves open: rsqrt is 1/sqrt correctly rounded, and a*b + c*d is not
contracted; the oracle makes the same two choices.
"""
import hashlib
import json
import os

import numpy as np
import pytest

import msl_cases
import msl_ref_lib as M
import oracle_lib as O

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden",
                                     "msl_scalar_kernels.json")))["cases"]


def check(key, out):
    out = np.ascontiguousarray(out, np.uint16)
    want = GOLDEN[key]
    assert out.size == want["elements"], key
    assert [int(v) for v in out.ravel()[:8]] == want["first8"], key
    assert hashlib.sha256(out.tobytes()).hexdigest() == want["sha256"], key


@pytest.mark.parametrize("seed", msl_cases.CASES["head_norm"])
@pytest.mark.parametrize("double_round", [0, 1])
def test_head_rms_norm_matches_shader(seed, double_round):
    x, w, s, h, eps = msl_cases.head_norm_case(seed)
    check(f"head_norm/{seed}/double_round={double_round}",
          O.head_rms_norm(x, w, s, h, eps, bool(double_round)))


@pytest.mark.parametrize("seed", msl_cases.CASES["rope"])
def test_rope_application_matches_shader(seed):
    q, k, cos, sin, s, h = msl_cases.rope_case(seed)
    qo, ko = O.qk_rope(q, k, cos, sin, s, h)
    check(f"rope/{seed}/q", qo)
    check(f"rope/{seed}/k", ko)


@pytest.mark.parametrize("seed,rows,width", msl_cases.CASES["rows"])
def test_layer_norm_mod_and_gate_match_shader(seed, rows, width):
    x, branch, mod, row_map, rows, width, slots = msl_cases.row_case(seed, rows, width)
    check(f"layer_norm_mod/{seed}/{rows}x{width}",
          O.layer_norm_mod(x, mod, row_map, rows, width, slots, 1, 1e-6))
    check(f"gate/{seed}/{rows}x{width}", O.gate(x, branch, mod, row_map, rows, width, slots, 2))


@pytest.mark.skipif(M.load() is None, reason="oracle/_ref/libmsl_ref.so not built here")
@pytest.mark.parametrize("seed", [101, 102, 103])
def test_oracle_equals_shader_build_on_fresh_seeds(seed):
    x, w, s, h, eps = msl_cases.head_norm_case(seed, sequence=64, heads=5)
    for dbl in (False, True):
        assert np.array_equal(O.head_rms_norm(x, w, s, h, eps, dbl),
                              M.head_rms_norm(x, w, s, h, eps, dbl))
    q, k, cos, sin, s, h = msl_cases.rope_case(seed, sequence=50, heads=4)
    oq, ok = O.qk_rope(q, k, cos, sin, s, h)
    mq, mk = M.qk_rope(q, k, cos, sin, s, h)
    assert np.array_equal(oq, mq) and np.array_equal(ok, mk)
    # in place, as the DiT block calls it (qwen_dit.m:1277)
    x, branch, mod, row_map, rows, width, slots = msl_cases.row_case(seed, 7, 3072)
    assert np.array_equal(O.layer_norm_mod(x, mod, row_map, rows, width, slots, 0, 1e-6),
                          M.layer_norm_mod(x, mod, row_map, rows, width, slots, 0, 1e-6))
    assert np.array_equal(O.gate(x, branch, mod, row_map, rows, width, slots, 3),
                          M.gate(x, branch, mod, row_map, rows, width, slots, 3))
