"""GPU parity of the block's AdaLN norm (qw_gpu_layer_norm_mod_bf16) and gated
residual (h3_gpu_gate_bf16) against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest

import oracle_lib as O
from qwen_metal_b200 import workloads

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16_steps(a_bits, b_bits):
    """Distance in bf16 steps between two arrays of bit patterns."""
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)
    return np.abs(key(a_bits) - key(b_bits))


def run_norm(gpu, x, mod, row_map, rows, width, slots, slot, eps=1e-6):
    xt, mt, rt, ot = gpu.bf16(x), gpu.bf16(mod), gpu.u32(row_map), gpu.new_bf16(rows * width)
    gpu.begin()
    gpu.check(gpu.lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, ot, xt, mt, rt, rows, width, slots,
                                                 slot, eps), "layer_norm_mod")
    gpu.submit()
    out = gpu.read_bf16(ot, rows * width).reshape(rows, width)
    for t in (xt, mt, rt, ot):
        gpu.free(t)
    return out


def run_gate(gpu, res, br, mod, row_map, rows, width, slots, slot, in_place=False):
    rt_, bt, mt, mapt = gpu.bf16(res), gpu.bf16(br), gpu.bf16(mod), gpu.u32(row_map)
    ot = rt_ if in_place else gpu.new_bf16(rows * width)
    gpu.begin()
    gpu.check(gpu.lib.h3_gpu_gate_bf16(gpu.handle, ot, rt_, bt, mt, mapt, rows, width, slots, slot),
              "gate")
    gpu.submit()
    out = gpu.read_bf16(ot, rows * width).reshape(rows, width)
    for t in {rt_, bt, mt, mapt, ot}:
        gpu.free(t)
    return out


def check_norm(got, ref):
    # The warp-tree sums differ from the oracle's serial sums in the last fp32 bits and
    # rsqrt is 1 ulp off 1/sqrt: a bf16 rounding flips by one step now and then.  Where
    # x - mean cancels to almost nothing, the few-ulp difference of the two means is a
    # large RELATIVE change of a tiny output: those are held to an absolute bound of
    # 1e-6 of the row's largest output instead (fp32 has 6e-8 per operation).
    d = bf16_steps(got, ref)
    a, b = O.bf16_to_f32(got), O.bf16_to_f32(ref)
    tiny = np.abs(a - b) <= 1e-6 * np.abs(b).max(axis=1, keepdims=True)
    assert ((d <= 1) | tiny).all(), int(d[~tiny].max())
    assert (d > 0).mean() < 5e-3, float((d > 0).mean())


def test_norm_mod_on_the_reference_block_fixture(gpu):
    stages = np.load(os.path.join(GOLD, "ref_block_stages.npz"))
    for case in "ab":
        x = stages[f"{case}_joint_in"]
        rows = x.shape[0]
        row_map = np.array([1 if i < int(stages[f"{case}_text_rows"]) else 0 for i in range(rows)],
                           np.uint32)
        mod = stages[f"{case}_modulation"]
        got = run_norm(gpu, x, mod, row_map, rows, 4096, 4, 0)
        check_norm(got, O.layer_norm_mod(x, mod, row_map, rows, 4096, 4, 0, 1e-6))
        a, b = O.bf16_to_f32(got).astype(np.float64), O.bf16_to_f32(stages[f"{case}_attn_in"]).astype(np.float64)
        assert np.sqrt(((a - b) ** 2).sum() / (b ** 2).sum()) < 2e-2  # the reference test's gate


@pytest.mark.parametrize("rows,width,slots,slot", [
    (8704, 3072, 4, 1),   # cfg3: batch 2 x 4352 rows, 24 heads x 128
    (4352, 4096, 4, 0),   # the model's own hidden size
    (149, 4096, 1, 0),    # final-norm form: one slot
    (37, 1000, 3, 2),     # width not a multiple of 8: plain loop
    (5, 8192, 2, 1),      # wider than the register copy: plain loop
    (3, 8, 1, 0),
])
def test_norm_mod_matches_oracle(gpu, rows, width, slots, slot):
    rng = np.random.default_rng(rows * 31 + width)
    x = workloads.normal_bf16(rng, (rows, width), 0.3, 1.7)
    maps = 3
    mod = workloads.normal_bf16(rng, (maps, slots, width), 0.0, 0.5)
    row_map = rng.integers(0, maps, rows).astype(np.uint32)
    got = run_norm(gpu, x, mod, row_map, rows, width, slots, slot)
    check_norm(got, O.layer_norm_mod(x, mod, row_map, rows, width, slots, slot, 1e-6))


@pytest.mark.parametrize("rows,width,slots,slot,in_place", [
    (8704, 3072, 4, 2, True),   # the block updates hidden in place (qwen_dit.m:1450)
    (4352, 4096, 4, 3, False),
    (37, 1000, 3, 0, False),
    (1, 8, 1, 0, True),
])
def test_gate_is_bit_exact(gpu, rows, width, slots, slot, in_place):
    rng = np.random.default_rng(rows * 17 + width)
    res = workloads.normal_bf16(rng, (rows, width))
    br = workloads.normal_bf16(rng, (rows, width))
    maps = 2
    mod = workloads.normal_bf16(rng, (maps, slots, width), 0.0, 0.5)
    row_map = rng.integers(0, maps, rows).astype(np.uint32)
    got = run_gate(gpu, res, br, mod, row_map, rows, width, slots, slot, in_place)
    # one fp32 product, one fp32 sum, one rounding: no freedom in the order
    assert np.array_equal(got, O.gate(res, br, mod, row_map, rows, width, slots, slot))


def test_rowwise_error_conventions(gpu):
    lib = gpu.lib
    x = gpu.new_bf16(64)
    m = gpu.new_bf16(64)
    r = gpu.u32(np.zeros(4, np.uint32))
    f = gpu.f32(np.zeros(64, np.float32))
    gpu.begin()
    assert not lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, x, x, m, r, 4, 16, 2, 2, 1e-6)  # slot >= slots
    assert not lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, x, x, m, r, 8, 8, 2, 0, 1e-6)   # row map too small
    assert "row map" in gpu.error()
    assert not lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, x, f, m, r, 4, 16, 2, 0, 1e-6)  # wrong dtype
    assert not lib.h3_gpu_gate_bf16(gpu.handle, x, x, x, m, r, 4, 16, 1, 1)               # slot >= slots
    assert not lib.h3_gpu_gate_bf16(gpu.handle, x, x, x, m, r, 4, 32, 1, 0)               # tensors too small
    assert lib.h3_gpu_gate_bf16(gpu.handle, x, x, x, m, r, 4, 16, 1, 0)
    gpu.submit()
    for t in (x, m, r, f):
        gpu.free(t)


def test_modulation_row_index_outside_the_tensor_is_reported(gpu):
    """row_map comes from device memory, so only the kernel can check it: an
    entry past the modulation tensor is reported at submit (no out-of-bounds
    read; block 0 stands in) and the context keeps working."""
    rng = np.random.default_rng(9)
    rows, width, slots = 8, 256, 4
    x = workloads.normal_bf16(rng, (rows, width))
    mod = workloads.normal_bf16(rng, (2, slots, width), 0.0, 0.5)
    row_map = np.array([0, 1, 0, 7, 1, 0, 1, 0], np.uint32)   # 7 >= 2 maps
    lib = gpu.lib
    xt, mt, rt, ot = gpu.bf16(x), gpu.bf16(mod), gpu.u32(row_map), gpu.new_bf16(rows * width)
    for call in ("norm", "gate"):
        gpu.begin()
        if call == "norm":
            gpu.check(lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, ot, xt, mt, rt, rows, width, slots,
                                                     1, 1e-6), "norm")
        else:
            gpu.check(lib.h3_gpu_gate_bf16(gpu.handle, ot, xt, xt, mt, rt, rows, width, slots, 2),
                      "gate")
        assert lib.h3_gpu_submit(gpu.handle) == 0
        assert "outside the modulation tensor" in gpu.error(), gpu.error()
        assert np.isfinite(O.bf16_to_f32(gpu.read_bf16(ot, rows * width))).all()
    # too small a modulation tensor is refused on the host
    small = gpu.bf16(mod.ravel()[:slots * width - 8])
    gpu.begin()
    assert lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, ot, xt, small, rt, rows, width, slots, 1,
                                          1e-6) == 0
    assert "less than one" in gpu.error()
    gpu.submit()
    good = np.zeros(rows, np.uint32)
    check_norm(run_norm(gpu, x, mod, good, rows, width, slots, 1),   # and the context still works
               O.layer_norm_mod(x, mod, good, rows, width, slots, 1, 1e-6))
    for t in (xt, mt, rt, ot, small):
        gpu.free(t)
