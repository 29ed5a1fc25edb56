"""ctypes access to the CPU oracle (oracle/libqw_oracle.so) for the tests.

The oracle is test infrastructure: it is built on demand from oracle/qw_oracle.c
and is never loaded by the product library.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB = os.path.join(ORACLE_DIR, "libqw_oracle.so")


class Segment(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("is_image", C.c_int), ("src_offset", C.c_uint32)]


_lib = None


def bf16_to_f32(bits):
    """bf16 bit patterns (uint16) as float32 values."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def load():
    global _lib
    if _lib is None:
        src = os.path.join(ORACLE_DIR, "qw_oracle.c")
        if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", ORACLE_DIR, "all"], stdout=subprocess.DEVNULL)
        lib = C.CDLL(LIB)
        lib.qwo_sdpa_prefix.restype = C.c_uint64
        lib.qwo_sdpa_prefix.argtypes = [C.c_void_p] * 5 + [C.c_int] + [C.c_uint32] * 6 + [
            C.c_float, C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t]
        lib.qwo_visible_pairs.restype = C.c_uint64
        lib.qwo_visible_pairs.argtypes = [C.c_void_p, C.c_int, C.c_uint32, C.c_uint32, C.c_uint32,
                                          C.c_void_p, C.c_uint32]
        lib.qwo_dense_mask.restype = None
        lib.qwo_dense_mask.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_uint32, C.c_uint32,
                                       C.c_uint32, C.c_void_p, C.c_uint32]
        lib.qwo_rope_tables.restype = C.c_uint32
        lib.qwo_rope_tables.argtypes = [C.c_uint32] * 3 + [C.c_void_p] * 2
        lib.qwo_rope_tables_blocks.restype = C.c_uint32
        lib.qwo_rope_tables_blocks.argtypes = [C.c_void_p] * 3 + [C.c_uint32] + [C.c_void_p] * 2
        lib.qwo_rope_released_entry.restype = None
        lib.qwo_rope_released_entry.argtypes = [C.c_int] * 3 + [C.POINTER(C.c_float)] * 2
        lib.qwo_head_rms_norm_bf16.restype = None
        lib.qwo_head_rms_norm_bf16.argtypes = [C.c_void_p, C.c_void_p] + [C.c_uint32] * 3 + [
            C.c_float, C.c_int]
        lib.qwo_qk_rope_bf16.restype = None
        lib.qwo_qk_rope_bf16.argtypes = [C.c_void_p] * 6 + [C.c_uint32] * 3
        lib.qwo_kat_fill.restype = None
        lib.qwo_layer_norm_mod_bf16.argtypes = [C.c_void_p] * 4 + [C.c_uint32] * 4 + [C.c_float]
        lib.qwo_layer_norm_mod_bf16.restype = None
        lib.qwo_gate_bf16.argtypes = [C.c_void_p] * 5 + [C.c_uint32] * 4
        lib.qwo_gate_bf16.restype = None
        lib.qwo_linear_bf16.restype = None
        lib.qwo_linear_bf16.argtypes = [C.c_void_p] * 4 + [C.c_uint32] * 3 + [C.c_void_p, C.c_size_t]
        lib.qwo_kat_fill.argtypes = [C.c_uint32] + [C.c_void_p] * 3 + [C.c_size_t]
        lib.qwo_kat_limits.restype = None
        lib.qwo_kat_limits.argtypes = [C.c_void_p]
        lib.qwo_prefix_limits.restype = None
        lib.qwo_prefix_limits.argtypes = [C.POINTER(Segment), C.c_uint32, C.c_void_p]
        lib.qwo_threads.restype = C.c_int
        _lib = lib
    return _lib


def threads():
    return load().qwo_threads()


def use_all_cores():
    """Let the oracle's OpenMP loops use every core this process may run on,
    whatever OMP_NUM_THREADS says (torchrun exports 1 to each rank)."""
    lib = load()
    lib.qwo_set_threads.argtypes = [C.c_int]
    lib.qwo_set_threads.restype = None
    lib.qwo_set_threads(len(os.sched_getaffinity(0)))
    return lib.qwo_threads()


def sdpa(q, k, v, limits, batch, q_rows, kv_rows, heads, kv_heads, scale, text_len=None,
         text_pad=0, rows=None, per_batch_limits=False):
    """fp32 oracle output [batch, q_rows, heads, 128]; `rows` = flat b*q_rows+r
    indices to compute (others stay 0), None = all.  Returns (out, visible)."""
    lib = load()
    out = np.zeros((batch, q_rows, heads, 128), dtype=np.float32)
    lim = None if limits is None else np.ascontiguousarray(limits, dtype=np.uint32)
    tl = None if text_len is None else np.ascontiguousarray(text_len, dtype=np.uint32)
    idx = None if rows is None else np.ascontiguousarray(rows, dtype=np.uint32)
    visible = lib.qwo_sdpa_prefix(_p(out), _p(np.ascontiguousarray(q)), _p(np.ascontiguousarray(k)),
                                  _p(np.ascontiguousarray(v)), _p(lim), int(per_batch_limits), batch,
                                  q_rows, kv_rows, heads, kv_heads, 128, scale, _p(tl), text_pad,
                                  _p(idx), 0 if idx is None else idx.size)
    return out, visible


def visible_pairs(limits, batch, q_rows, kv_rows, text_len=None, text_pad=0, per_batch=False):
    lib = load()
    lim = None if limits is None else np.ascontiguousarray(limits, dtype=np.uint32)
    tl = None if text_len is None else np.ascontiguousarray(text_len, dtype=np.uint32)
    return lib.qwo_visible_pairs(_p(lim), int(per_batch), batch, q_rows, kv_rows, _p(tl), text_pad)


def dense_mask(limits, batch, rows, kv_rows, text_len=None, text_pad=0, per_batch=False):
    lib = load()
    mask = np.zeros((batch, rows, kv_rows), dtype=np.uint8)
    lim = None if limits is None else np.ascontiguousarray(limits, dtype=np.uint32)
    tl = None if text_len is None else np.ascontiguousarray(text_len, dtype=np.uint32)
    lib.qwo_dense_mask(_p(mask), _p(lim), int(per_batch), batch, rows, kv_rows, _p(tl), text_pad)
    return mask


def rope_tables(text_rows, gh, gw):
    lib = load()
    rows = text_rows + gh * gw
    cos = np.empty((rows, 64), np.float32)
    sin = np.empty((rows, 64), np.float32)
    assert lib.qwo_rope_tables(text_rows, gh, gw, _p(cos), _p(sin)) == rows
    return cos, sin


def rope_tables_blocks(block_h, block_w, text_before):
    lib = load()
    bh, bw, tb = (np.asarray(x, dtype=np.uint32) for x in (block_h, block_w, text_before))
    rows = int((tb + bh * bw).sum())
    cos = np.empty((rows, 64), np.float32)
    sin = np.empty((rows, 64), np.float32)
    assert lib.qwo_rope_tables_blocks(_p(bh), _p(bw), _p(tb), len(bh), _p(cos), _p(sin)) == rows
    return cos, sin


def released_entry(axis_dim, pair, coordinate):
    lib = load()
    c, s = C.c_float(), C.c_float()
    lib.qwo_rope_released_entry(axis_dim, pair, coordinate, C.byref(c), C.byref(s))
    return c.value, s.value


def head_rms_norm(x, weight, sequence, heads, eps, double_round=False):
    lib = load()
    out = np.array(x, dtype=np.uint16, copy=True)
    lib.qwo_head_rms_norm_bf16(_p(out), _p(np.ascontiguousarray(weight, dtype=np.uint16)),
                               sequence, heads, 128, eps, int(double_round))
    return out


def layer_norm_mod(x, modulation, row_map, rows, width, slots, scale_slot, eps):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    modulation = np.ascontiguousarray(modulation, dtype=np.uint16)
    row_map = np.ascontiguousarray(row_map, dtype=np.uint32)
    out = np.empty(rows * width, np.uint16)
    load().qwo_layer_norm_mod_bf16(_p(out), _p(x), _p(modulation), _p(row_map), rows, width,
                                   slots, scale_slot, eps)
    return out.reshape(rows, width)


def gate(residual, branch, modulation, row_map, rows, width, slots, gate_slot):
    residual = np.ascontiguousarray(residual, dtype=np.uint16)
    branch = np.ascontiguousarray(branch, dtype=np.uint16)
    modulation = np.ascontiguousarray(modulation, dtype=np.uint16)
    row_map = np.ascontiguousarray(row_map, dtype=np.uint32)
    out = np.empty(rows * width, np.uint16)
    load().qwo_gate_bf16(_p(out), _p(residual), _p(branch), _p(modulation), _p(row_map), rows,
                         width, slots, gate_slot)
    return out.reshape(rows, width)


def qk_rope(q, k, cos, sin, sequence, heads):
    lib = load()
    qo = np.empty_like(q)
    ko = np.empty_like(k)
    lib.qwo_qk_rope_bf16(_p(qo), _p(ko), _p(np.ascontiguousarray(q)), _p(np.ascontiguousarray(k)),
                         _p(np.ascontiguousarray(cos, dtype=np.float32)),
                         _p(np.ascontiguousarray(sin, dtype=np.float32)), sequence, heads, 128)
    return qo, ko


def kat_inputs(seed=20261028, rows=149, heads=32):
    lib = load()
    n = rows * heads * 128
    q, k, v = (np.empty(n, np.uint16) for _ in range(3))
    lib.qwo_kat_fill(seed, _p(q), _p(k), _p(v), n)
    limits = np.empty(149, np.uint32)
    lib.qwo_kat_limits(_p(limits))
    return q, k, v, limits


def prefix_limits(segments):
    lib = load()
    arr = (Segment * len(segments))(*[Segment(r, int(i), 0) for r, i in segments])
    out = np.zeros(sum(r for r, _ in segments), np.uint32)
    lib.qwo_prefix_limits(arr, len(segments), _p(out))
    return out


def linear(x, weight, bias, rows, input_dim, output_dim, row_index=None):
    """bf16 linear layer (bits in, bits out); row_index = rows to compute (others 0)."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    weight = np.ascontiguousarray(weight, dtype=np.uint16)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.uint16)
    idx = None if row_index is None else np.ascontiguousarray(row_index, dtype=np.uint32)
    out = np.zeros(rows * output_dim, np.uint16)
    load().qwo_linear_bf16(_p(out), _p(x), _p(weight), _p(b), rows, input_dim, output_dim, _p(idx),
                           0 if idx is None else idx.size)
    return out.reshape(rows, output_dim)
