"""GPU: h3_gpu_gqa_causal_noalloc_bf16, the causal attention op for callers that
cannot allocate device memory when they call it (a host whose own arena owns
the whole GPU, or a loop that must not stall on an allocation).  It must give
exactly what h3_gpu_gqa_causal_bf16 gives, call after call, although every call
reuses one fixed scratch array that still holds the previous call's bytes.

Collected last on purpose: a failure here leaves every other test already run.
"""
import numpy as np
import pytest

import oracle_lib as O
from qwen_metal_b200 import abi, workloads
from qwen_metal_b200.abi import bf16_to_f32, f32_to_bf16

pytestmark = pytest.mark.gpu

SCALE = workloads.SCALE


def both_ops(gpu, q, k, v, S, QH, KVH):
    lib = gpu.lib
    qt, kt, vt = gpu.bf16(q), gpu.bf16(k), gpu.bf16(v)
    regular, fixed = gpu.new_bf16(q.size), gpu.new_bf16(q.size)
    gpu.begin()
    gpu.check(lib.h3_gpu_gqa_causal_bf16(gpu.handle, regular, qt, kt, vt, S, QH, KVH, 128, SCALE),
              "regular op")
    gpu.check(lib.h3_gpu_gqa_causal_noalloc_bf16(gpu.handle, fixed, qt, kt, vt, S, QH, KVH, 128,
                                                 SCALE), "no-alloc op")
    gpu.submit()
    a = gpu.read_bf16(regular, q.size).reshape(q.shape)
    b = gpu.read_bf16(fixed, q.size).reshape(q.shape)
    for t in (qt, kt, vt, regular, fixed):
        gpu.free(t)
    return a, b


def test_noalloc_matches_regular_op_on_two_calls_in_a_row(gpu):
    rng = np.random.default_rng(2026)
    # second call is smaller: the tail of the scratch still holds the first call's query
    for S, QH, KVH in ((384, 8, 2), (150, 4, 4)):
        q = workloads.normal_bf16(rng, (S, QH, 128))
        k = workloads.normal_bf16(rng, (S, KVH, 128))
        v = workloads.normal_bf16(rng, (S, KVH, 128))
        regular, fixed = both_ops(gpu, q, k, v, S, QH, KVH)
        # tolerance of the parity tests (max-abs 2e-2, mean-abs 2e-3, relL2 5e-3) ...
        got, ref = bf16_to_f32(fixed).astype(np.float64), bf16_to_f32(regular).astype(np.float64)
        diff = np.abs(got - ref)
        assert diff.max() <= 2e-2 and diff.mean() <= 2e-3
        assert np.sqrt((diff ** 2).sum() / (ref ** 2).sum()) < 5e-3
        # ... and in fact the same bits: both run the same arithmetic
        assert np.array_equal(regular, fixed)
        # and both agree with the CPU oracle of the pre-scaled-query variant
        q_scaled = f32_to_bf16(bf16_to_f32(q) * np.float32(SCALE))
        oracle, _ = O.sdpa(q_scaled, k, v, np.arange(1, S + 1, dtype=np.uint32), 1, S, S, QH, KVH, 1.0)
        d = np.abs(got - oracle[0])
        assert d.max() <= 2e-2 and d.mean() <= 2e-3


def test_noalloc_rejects_oversize_and_bad_scale(gpu):
    lib = gpu.lib
    t = gpu.new_bf16(128)
    gpu.begin()
    # 4097 * 8 * 128 > 4,194,304 elements of fixed scratch
    assert lib.h3_gpu_gqa_causal_noalloc_bf16(gpu.handle, t, t, t, t, 4097, 8, 8, 128, SCALE) == 0
    assert "exceeds the fixed scratch" in gpu.error()
    assert lib.h3_gpu_gqa_causal_noalloc_bf16(gpu.handle, t, t, t, t, 1, 1, 1, 128, 0.0) == 0
    assert "scale must be positive" in gpu.error()
    assert lib.h3_gpu_gqa_causal_noalloc_bf16(gpu.handle, t, t, t, t, 1, 1, 1, 64, SCALE) == 0
    assert "unsupported geometry" in gpu.error()
    gpu.submit()
    gpu.free(t)
