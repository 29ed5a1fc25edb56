"""GPU parity of the linear layers either side of the attention path: the output
projection (h3_gpu_linear_bf16), the fused q/k/v projection (qw_gpu_qkv_bf16) and
the q/k/v projection with the QK-norm + RoPE in its epilogue
(qw_gpu_qkv_norm_rope_bf16), through the C ABI, against the CPU oracle.

Tolerance of the GEMM itself: the tensor cores accumulate in fp32 in an order of
their own while the oracle runs the reference's serial fma chain, so a result may
land on the neighbouring bf16 value: at most 1 bf16 step apart (2 where the value
sits next to a power of two), relL2 < 3e-3.  The fused epilogue is checked bit for
bit: it must equal the oracle's norm + rotation applied to the plain GEMM's own
bf16 output.
"""
import numpy as np
import pytest

import oracle_lib as O
from qwen_metal_b200 import abi, workloads
from qwen_metal_b200.abi import bf16_to_f32

pytestmark = pytest.mark.gpu


def bf16_steps(a_bits, b_bits):
    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)
    return np.abs(key(a_bits) - key(b_bits))


def check_gemm(got, ref, what):
    a, b = bf16_to_f32(got).astype(np.float64), bf16_to_f32(ref).astype(np.float64)
    assert np.isfinite(a).all(), what
    rel = np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-30))
    assert rel < 3e-3, (what, rel)
    d = bf16_steps(np.asarray(got), np.asarray(ref))
    # values near zero have tiny steps: hold those to an absolute bound instead
    small = np.abs(a - b) <= 2e-3 * np.abs(b).max()
    assert ((d <= 2) | small).all(), (what, int(d[~small].max()))


def weights(rng, n, k):
    return workloads.normal_bf16(rng, (n, k), 0.0, 1.0 / np.sqrt(k))


@pytest.mark.parametrize("rows,k,n,with_bias", [(300, 512, 768, True), (129, 72, 264, False),
                                                 (1024, 3072, 3072, False)])
def test_linear_matches_oracle(gpu, rows, k, n, with_bias):
    """Output projection: ragged rows (not a tile multiple), a K tail (72 = 64 + 8),
    an N tail (264 = 256 + 8), bias, and the DiT shape on a row sample."""
    rng = np.random.default_rng(rows + k)
    x, w = workloads.normal_bf16(rng, (rows, k)), weights(rng, n, k)
    bias = workloads.normal_bf16(rng, (n,)) if with_bias else None
    xt, wt, ot = gpu.bf16(x), gpu.bf16(w), gpu.new_bf16(rows * n)
    bt = gpu.bf16(bias) if with_bias else None
    gpu.begin()
    gpu.check(gpu.lib.h3_gpu_linear_bf16(gpu.handle, ot, xt, wt, bt, rows, k, n), "linear")
    gpu.submit()
    got = gpu.read_bf16(ot, rows * n).reshape(rows, n)
    sample = None if rows * k * n < 2e9 else np.unique(
        np.concatenate([[0, 1, 127, 128, rows - 1], rng.integers(0, rows, 96)])).astype(np.uint32)
    ref = O.linear(x, w, bias, rows, k, n, sample)
    if sample is None:
        check_gemm(got, ref, f"linear {rows}x{k}x{n}")
    else:
        check_gemm(got[sample], ref[sample], f"linear {rows}x{k}x{n} (row sample)")
    for t in [xt, wt, ot] + ([bt] if bt else []):
        gpu.free(t)


def test_linear_error_conventions(gpu):
    lib = gpu.lib
    t = gpu.new_bf16(64 * 64)
    f = gpu.new_f32(64 * 64)
    assert lib.h3_gpu_linear_bf16(gpu.handle, t, t, t, None, 8, 64, 64) == 0
    assert "h3_gpu_begin() was not called" in gpu.error()
    gpu.begin()
    assert lib.h3_gpu_linear_bf16(gpu.handle, t, t, t, None, 128, 64, 64) == 0
    assert "absent or too small" in gpu.error()
    assert lib.h3_gpu_linear_bf16(gpu.handle, t, f, t, None, 8, 64, 64) == 0
    assert "not BF16" in gpu.error()
    assert lib.h3_gpu_linear_bf16(gpu.handle, t, t, t, None, 8, 60, 64) == 0
    assert "unsupported geometry" in gpu.error()
    gpu.submit()
    gpu.free(t), gpu.free(f)


@pytest.mark.parametrize("batch,seq,dim", [(1, 200, 512), (2, 333, 768)])
def test_qkv_and_fused_norm_rope_epilogue(gpu, batch, seq, dim):
    """qw_gpu_qkv_bf16 against the oracle GEMM; then the fused epilogue against the
    reference's own sequence (QKV -> head RMSNorm x2 -> RoPE, qwen_dit.m:1270-1278)
    run by the oracle on the plain GEMM's bf16 output: bit for bit, v untouched, and
    the score bound equals the prologue kernel's."""
    rng = np.random.default_rng(dim + seq)
    lib = gpu.lib
    rows, heads = batch * seq, dim // 128
    x = workloads.normal_bf16(rng, (rows, dim))
    ws = [weights(rng, dim, dim) for _ in range(3)]
    wq, wk = workloads.normal_bf16(rng, (128,), 1.0, 0.1), workloads.normal_bf16(rng, (128,), 1.0, 0.1)
    cos, sin = abi.rope_tables(seq - 144, 12, 12)
    xt = gpu.bf16(x)
    wts = [gpu.bf16(w) for w in ws]
    plain = [gpu.new_bf16(rows * dim) for _ in range(3)]
    fused = [gpu.new_bf16(rows * dim) for _ in range(3)]
    wqt, wkt, ct, st, bt = gpu.bf16(wq), gpu.bf16(wk), gpu.f32(cos), gpu.f32(sin), gpu.new_f32(2)
    gpu.begin()
    gpu.check(lib.qw_gpu_qkv_bf16(gpu.handle, *plain, xt, *wts, rows, dim), "qkv")
    gpu.check(lib.qw_gpu_qkv_norm_rope_bf16(gpu.handle, *fused, xt, *wts, wqt, wkt, ct, st, bt,
                                            batch, seq, dim, 1e-6), "qkv norm rope")
    gpu.submit()
    got = [gpu.read_bf16(t, rows * dim).reshape(rows, dim) for t in plain]
    for name, g, w in zip("qkv", got, ws):
        check_gemm(g, O.linear(x, w, None, rows, dim, dim), f"qkv {name}")
    qn = O.head_rms_norm(got[0].reshape(rows, heads, 128), wq, rows, heads, 1e-6)
    kn = O.head_rms_norm(got[1].reshape(rows, heads, 128), wk, rows, heads, 1e-6)
    want_q, want_k = np.empty_like(qn), np.empty_like(kn)
    for b in range(batch):
        sl = slice(b * seq, (b + 1) * seq)
        want_q[sl], want_k[sl] = O.qk_rope(qn[sl], kn[sl], cos, sin, seq, heads)
    fq, fk, fv = (gpu.read_bf16(t, rows * dim).reshape(rows, heads, 128) for t in fused)
    assert np.array_equal(fv.reshape(rows, dim), got[2])          # v: the plain GEMM
    assert np.array_equal(fq, want_q), float((fq != want_q).mean())
    assert np.array_equal(fk, want_k), float((fk != want_k).mean())
    bound = gpu.read_f32(bt, 2)
    assert np.sqrt((bf16_to_f32(fq).astype(np.float64) ** 2).sum(-1)).max() <= bound[0]
    assert np.sqrt((bf16_to_f32(fk).astype(np.float64) ** 2).sum(-1)).max() <= bound[1]
    for t in [xt, wqt, wkt, ct, st, bt] + wts + plain + fused:
        gpu.free(t)
