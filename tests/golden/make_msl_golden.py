#!/usr/bin/env python3
"""Golden outputs of the reference's scalar shader kernels of the attention path.

    make -C oracle ref REF=<reference checkout>     # builds oracle/_ref/libmsl_ref.so
    python tests/golden/make_msl_golden.py

Runs the shader-built kernels (the reference's text compiled as C++, see
oracle/msl_shim.h) on the seeded cases of tests/msl_cases.py and records, per
case and kernel, the SHA-256 of the bf16 output bytes and its first values in
tests/golden/msl_scalar_kernels.json.  The CPU test holds the oracle to these
bit for bit, with or without a reference checkout.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import msl_cases  # noqa: E402
import msl_ref_lib as M  # noqa: E402


def record(out):
    out = np.ascontiguousarray(out, np.uint16)
    return {"sha256": hashlib.sha256(out.tobytes()).hexdigest(), "elements": int(out.size),
            "first8": [int(v) for v in out.ravel()[:8]]}


def main():
    if M.load() is None:
        sys.exit("oracle/_ref/libmsl_ref.so is missing: run `make -C oracle ref` first")
    golden = {"source": "h3_shaders.metal kernels h3_head_rms_norm_bf16, qw_head_rms_norm_bf16, "
                        "qw_qk_rope_bf16, qw_layer_norm_mod_bf16 (256 threads per row), "
                        "h3_gate_bf16, compiled as C++ (oracle/msl_shim.h)",
              "cases": {}}
    for seed in msl_cases.CASES["head_norm"]:
        x, w, s, h, eps = msl_cases.head_norm_case(seed)
        for dbl in (0, 1):
            golden["cases"][f"head_norm/{seed}/double_round={dbl}"] = record(
                M.head_rms_norm(x, w, s, h, eps, dbl))
    for seed in msl_cases.CASES["rope"]:
        q, k, cos, sin, s, h = msl_cases.rope_case(seed)
        qo, ko = M.qk_rope(q, k, cos, sin, s, h)
        golden["cases"][f"rope/{seed}/q"] = record(qo)
        golden["cases"][f"rope/{seed}/k"] = record(ko)
    for seed, rows, width in msl_cases.CASES["rows"]:
        x, branch, mod, row_map, rows, width, slots = msl_cases.row_case(seed, rows, width)
        golden["cases"][f"layer_norm_mod/{seed}/{rows}x{width}"] = record(
            M.layer_norm_mod(x, mod, row_map, rows, width, slots, 1, 1e-6))
        golden["cases"][f"gate/{seed}/{rows}x{width}"] = record(
            M.gate(x, branch, mod, row_map, rows, width, slots, 2))
    path = os.path.join(HERE, "msl_scalar_kernels.json")
    json.dump(golden, open(path, "w"), indent=1)
    print("wrote", path, len(golden["cases"]), "cases")


if __name__ == "__main__":
    main()
