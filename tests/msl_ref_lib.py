"""ctypes access to oracle/_ref/libmsl_ref.so: the reference's own scalar shader
kernels (head RMSNorm x2, interleaved RoPE, AdaLN norm, gated residual) compiled
as C++ from the reference's shader text (`make -C oracle ref`).  Present only
where a reference checkout was available at build time; load() returns None
otherwise.  Test infrastructure only.
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "_ref", "libmsl_ref.so")

_lib = None


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def load():
    global _lib
    if _lib is None and os.path.exists(LIB):
        lib = C.CDLL(LIB)
        u32, f32 = C.c_uint32, C.c_float
        lib.msl_head_rms_norm_bf16.argtypes = [C.c_void_p, C.c_void_p, u32, u32, u32, f32, C.c_int]
        lib.msl_qk_rope_bf16.argtypes = [C.c_void_p] * 6 + [u32] * 3
        lib.msl_layer_norm_mod_bf16.argtypes = [C.c_void_p] * 4 + [u32] * 4 + [f32, u32]
        lib.msl_gate_bf16.argtypes = [C.c_void_p] * 5 + [u32] * 4
        for fn in (lib.msl_head_rms_norm_bf16, lib.msl_qk_rope_bf16, lib.msl_layer_norm_mod_bf16,
                   lib.msl_gate_bf16):
            fn.restype = None
        _lib = lib
    return _lib


def head_rms_norm(x, weight, sequence, heads, eps, double_round=False):
    out = np.array(x, dtype=np.uint16, copy=True)
    load().msl_head_rms_norm_bf16(_p(out), _p(np.ascontiguousarray(weight, np.uint16)), sequence,
                                  heads, 128, eps, int(double_round))
    return out


def qk_rope(q, k, cos, sin, sequence, heads):
    q, k = np.ascontiguousarray(q, np.uint16), np.ascontiguousarray(k, np.uint16)
    qo, ko = np.empty_like(q), np.empty_like(k)
    load().msl_qk_rope_bf16(_p(qo), _p(ko), _p(q), _p(k), _p(np.ascontiguousarray(cos, np.float32)),
                            _p(np.ascontiguousarray(sin, np.float32)), sequence, heads, 128)
    return qo, ko


def layer_norm_mod(x, modulation, row_map, rows, width, slots, scale_slot, eps, threads=256):
    x = np.ascontiguousarray(x, np.uint16)
    out = np.empty(rows * width, np.uint16)
    load().msl_layer_norm_mod_bf16(_p(out), _p(x), _p(np.ascontiguousarray(modulation, np.uint16)),
                                   _p(np.ascontiguousarray(row_map, np.uint32)), rows, width,
                                   slots, scale_slot, eps, threads)
    return out.reshape(rows, width)


def gate(residual, branch, modulation, row_map, rows, width, slots, gate_slot):
    out = np.empty(rows * width, np.uint16)
    load().msl_gate_bf16(_p(out), _p(np.ascontiguousarray(residual, np.uint16)),
                         _p(np.ascontiguousarray(branch, np.uint16)),
                         _p(np.ascontiguousarray(modulation, np.uint16)),
                         _p(np.ascontiguousarray(row_map, np.uint32)), rows, width, slots,
                         gate_slot)
    return out.reshape(rows, width)
