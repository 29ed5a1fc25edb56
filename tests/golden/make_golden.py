#!/usr/bin/env python3
"""Regenerate the golden fixtures under tests/golden/ from a reference checkout.

Run where a checkout of the reference project is present (--ref names it; see the
default below):

    python tests/golden/make_golden.py [--ref <checkout>]

It writes only small data files next to this script:

  ref_rope_tables.npz      the reference's own RoPE table fixtures, verbatim:
                           tests/pipeline_fixture/rope_{cos,sin}_{4,8}.f32 (text 23,
                           grids 4x4 and 8x8; tests/test_pipeline.c:68-124) and
                           tests/dit_fixture/{a,b,c}_rope_{cos,sin}.f32 with the row
                           layout from tests/dit_fixture/meta.json
  host_ref_rope.json       the 144 released-table samples of tests/host_ref.h:19-57
  dit_segments.json        run layout of fixture case c (tests/dit_fixture/meta.json)
  reference_abi_names.json the function names declared by h3_gpu.h and qwen_gpu_ext.h
  ref_block_stages.npz     stage tensors of the reference's DiT block fixture
                           (tests/dit_fixture/{a,b}_*.bin, bf16 [rows, 4096]; the stages
                           tests/test_dit_block.c:204-212 compares) around the AdaLN norm
                           and the gated residual: joint_in, modulation [2,4,4096], attn_in
                           for cases a and b; attn_out, mlp_in, mlp_out, block_out for b
  kat_prefix_sdpa.json     verdict of the reference's tests/test_prefix_kernel.c
                           compiled unmodified with the CPU oracle behind the op
                           (oracle/_ref/test_prefix_kernel_oracle), plus a checksum of
                           the oracle's fp32 output for that input

The GPU box has no reference checkout; tests read these files only.
"""
import argparse
import hashlib
import json
import os
import re
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def f32(path):
    return np.fromfile(path, dtype="<f4")


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--ref", default=os.environ.get("QWEN_METAL_REF") or
                        os.path.join(os.path.dirname(ROOT), "reference"))
    args = parser.parse_args()
    ref = args.ref
    if not os.path.isdir(ref):
        sys.exit(f"reference checkout not found at {ref}")

    tables = {}
    for grid in (4, 8):
        for kind in ("cos", "sin"):
            data = f32(os.path.join(ref, "tests/pipeline_fixture", f"rope_{kind}_{grid}.f32"))
            tables[f"pipeline_{kind}_{grid}"] = data.reshape(-1, 64)
    for case in "abc":
        for kind in ("cos", "sin"):
            data = f32(os.path.join(ref, "tests/dit_fixture", f"{case}_rope_{kind}.f32"))
            tables[f"dit_{case}_{kind}"] = data.reshape(-1, 64)
    np.savez_compressed(os.path.join(HERE, "ref_rope_tables.npz"), **tables)

    header = open(os.path.join(ref, "tests/host_ref.h")).read()
    body = header[header.index("host_ref_rope_samples"):]
    samples = [
        [int(a), int(r), int(p), float(c), float(s)]
        for a, r, p, c, s in re.findall(
            r"\{(\d+), (\d+), (\d+), (-?[0-9.e+-]+)f, (-?[0-9.e+-]+)f\}", body)
    ]
    assert len(samples) == 144, len(samples)
    json.dump({"source": "tests/host_ref.h:19-57", "axis_dim": [16, 56, 56],
               "pos_rows": 8192, "neg_rows": 1024,
               "samples": samples},
              open(os.path.join(HERE, "host_ref_rope.json"), "w"))

    meta = json.load(open(os.path.join(ref, "tests/dit_fixture/meta.json")))
    json.dump({"source": "tests/dit_fixture/meta.json",
               "heads": meta["heads"], "head_dim": meta["head_dim"], "eps": meta["eps"],
               "cases": meta["cases"]},
              open(os.path.join(HERE, "dit_segments.json"), "w"))

    stages = {}
    for case, names in (("a", ("joint_in", "modulation", "attn_in")),
                        ("b", ("joint_in", "modulation", "attn_in", "attn_out", "mlp_in",
                               "mlp_out", "block_out"))):
        for name in names:
            data = np.fromfile(os.path.join(ref, "tests/dit_fixture", f"{case}_{name}.bin"),
                               dtype="<u2")
            stages[f"{case}_{name}"] = data.reshape(-1, meta["hidden"])
        stages[f"{case}_text_rows"] = np.array(meta["cases"][case]["text_rows"], np.uint32)
    np.savez_compressed(os.path.join(HERE, "ref_block_stages.npz"), **stages)

    # every function name the two ABI headers declare (names only)
    abi_names = set()
    for header in ("h3_gpu.h", "qwen_gpu_ext.h"):
        text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ref, header)).read(), flags=re.S)
        abi_names |= set(re.findall(r"\b((?:h3_gpu|qw_gpu)_\w+)\s*\(", text))
    json.dump({"source": "h3_gpu.h, qwen_gpu_ext.h (declared function names)",
               "names": sorted(abi_names)},
              open(os.path.join(HERE, "reference_abi_names.json"), "w"))

    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "all", "ref", f"REF={ref}"],
                          stdout=subprocess.DEVNULL)
    with tempfile.TemporaryDirectory() as tmp:
        dump = os.path.join(tmp, "out.f32")
        env = dict(os.environ, QWO_SHIM_DUMP_F32=dump)
        out = subprocess.run([os.path.join(ROOT, "oracle/_ref/test_prefix_kernel_oracle")],
                             env=env, capture_output=True, text=True, check=True).stdout
        result = f32(dump)
    rel = float(re.search(r"relL2 ([0-9.e+-]+)", out).group(1))
    json.dump({
        "source": "tests/test_prefix_kernel.c (unmodified) + oracle behind the op",
        "seed": 20261028, "rows": 149, "heads": 32, "head_dim": 128,
        "relL2_vs_reference_cpu_loop": rel, "gate": 5e-3,
        "verdict": "PASS" if "PASS" in out else "FAIL",
        "oracle_output_sha256": hashlib.sha256(result.tobytes()).hexdigest(),
        "oracle_output_abs_sum": float(np.abs(result.astype(np.float64)).sum()),
        "oracle_output_first8": [float(x) for x in result[:8]],
    }, open(os.path.join(HERE, "kat_prefix_sdpa.json"), "w"), indent=1)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
