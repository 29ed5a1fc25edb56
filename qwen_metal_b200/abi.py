"""ctypes binding of libqwen_attn_b200.so (the C ABI declared in include/*.h).

This is the Python stub a test or benchmark uses to reach the library; it adds
no compute of its own.  bf16 tensors travel as numpy uint16 arrays, limits as
uint32, tables as float32.  The library is loaded from qwen_metal_b200/lib/ and
loading fails loudly when it has not been built (there is no fallback path).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# QWEN_METAL_B200_LIB points at another build of the library (e.g. one compiled
# with tracing); by default the in-tree build is loaded.
LIB_PATH = os.environ.get("QWEN_METAL_B200_LIB") or os.path.join(_HERE, "lib", "libqwen_attn_b200.so")

c_gpu = C.c_void_p
c_tensor = C.c_void_p
u32 = C.c_uint32
f32 = C.c_float
size_t = C.c_size_t

F32, BF16, I8, U32 = 0, 1, 2, 3


class Segment(C.Structure):
    """qw_dit_segment (reference qwen_dit.h:25-29)."""
    _fields_ = [("rows", u32), ("is_image", C.c_int), ("src_offset", u32)]


class Stats(C.Structure):
    """h3_gpu_stats (reference h3_gpu.h:21-37)."""
    _fields_ = [(n, C.c_uint64) for n in (
        "allocated_bytes", "live_bytes", "peak_live_bytes", "tensor_allocations",
        "direct_dispatches", "mps_linear_dispatches", "mps_conv_dispatches",
        "mps_sdpa_dispatches", "blit_copies", "submissions")] + [
        (n, C.c_double) for n in ("command_encode_seconds", "command_wait_seconds", "gpu_seconds")]


_SIGNATURES = {
    # name: (restype, argtypes)
    "h3_gpu_create": (c_gpu, [C.c_char_p, C.c_char_p, size_t]),
    "qw_gpu_create_on_device": (c_gpu, [C.c_int, C.c_char_p, size_t]),
    "h3_gpu_free": (None, [c_gpu]),
    "h3_gpu_is_m5": (C.c_int, [c_gpu]),
    "h3_gpu_has_nax_mlp": (C.c_int, [c_gpu]),
    "h3_gpu_has_int8_mlp": (C.c_int, [c_gpu]),
    "h3_gpu_clear_graph_cache": (None, [c_gpu]),
    "h3_gpu_tensor_new_f32": (c_tensor, [c_gpu, size_t]),
    "h3_gpu_tensor_new_bf16": (c_tensor, [c_gpu, size_t]),
    "h3_gpu_tensor_new_i8": (c_tensor, [c_gpu, size_t]),
    "h3_gpu_tensor_from_f32": (c_tensor, [c_gpu, C.c_void_p, size_t]),
    "h3_gpu_tensor_from_bf16": (c_tensor, [c_gpu, C.c_void_p, size_t]),
    "h3_gpu_tensor_from_u32": (c_tensor, [c_gpu, C.c_void_p, size_t]),
    "h3_gpu_tensor_free": (None, [c_tensor]),
    "h3_gpu_tensor_elements": (size_t, [c_tensor]),
    "h3_gpu_tensor_dtype": (C.c_int, [c_tensor]),
    "h3_gpu_tensor_read_f32": (C.c_int, [c_tensor, C.c_void_p, size_t]),
    "h3_gpu_tensor_read_f32_range": (C.c_int, [c_tensor, size_t, C.c_void_p, size_t]),
    "h3_gpu_tensor_read_bf16": (C.c_int, [c_tensor, C.c_void_p, size_t]),
    "h3_gpu_tensor_write_f32": (C.c_int, [c_tensor, C.c_void_p, size_t]),
    "h3_gpu_tensor_write_f32_range": (C.c_int, [c_tensor, size_t, C.c_void_p, size_t]),
    "h3_gpu_tensor_write_bf16": (C.c_int, [c_tensor, C.c_void_p, size_t]),
    "h3_gpu_tensor_write_bf16_range": (C.c_int, [c_tensor, size_t, C.c_void_p, size_t]),
    "h3_gpu_begin": (C.c_int, [c_gpu]),
    "h3_gpu_continue": (C.c_int, [c_gpu]),
    "h3_gpu_submit": (C.c_int, [c_gpu]),
    "h3_gpu_error": (C.c_char_p, [c_gpu]),
    "h3_gpu_get_stats": (C.c_int, [c_gpu, C.POINTER(Stats)]),
    "h3_gpu_profile_set_label": (None, [c_gpu, C.c_char_p]),
    "h3_gpu_profile_mark": (None, [c_gpu, C.c_char_p]),
    "h3_gpu_copy_bf16": (C.c_int, [c_gpu, c_tensor, size_t, c_tensor, size_t, size_t]),
    "h3_gpu_copy_f32": (C.c_int, [c_gpu, c_tensor, size_t, c_tensor, size_t, size_t]),
    "h3_gpu_sdpa_bf16": (C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, f32]),
    "h3_gpu_sdpa_bf16_head_major_output": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, f32]),
    "h3_gpu_head_rms_norm_bf16": (C.c_int, [c_gpu, c_tensor, c_tensor, u32, u32, u32, f32]),
    "h3_gpu_linear_bf16": (C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32]),
    "qw_gpu_qkv_bf16": (C.c_int, [c_gpu] + [c_tensor] * 7 + [u32, u32]),
    "qw_gpu_qkv_norm_rope_bf16": (C.c_int, [c_gpu] + [c_tensor] * 12 + [u32, u32, u32, f32]),
    "h3_gpu_gate_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32]),
    "h3_gpu_gqa_causal_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, f32]),
    "h3_gpu_gqa_causal_noalloc_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, f32]),
    "qw_gpu_qk_rope_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32]),
    "qw_gpu_head_rms_norm_bf16": (C.c_int, [c_gpu, c_tensor, c_tensor, u32, u32, u32, f32]),
    "qw_gpu_layer_norm_mod_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, f32]),
    "qw_gpu_flash_sdpa_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, f32]),
    "qw_gpu_flash_sdpa_prefix_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, u32, f32]),
    "qw_gpu_gqa_causal_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, f32]),
    "qw_gpu_sdpa_rect_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, f32]),
    "qw_gpu_qk_norm_rope_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor,
                  u32, u32, u32, u32, f32]),
    "qw_gpu_qk_norm_rope_out_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor,
                  c_tensor, u32, u32, u32, u32, f32]),
    "qw_gpu_qk_norm_rope_bound_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor,
                  c_tensor, c_tensor, u32, u32, u32, u32, f32]),
    "qw_gpu_attn_block_causal_bounded_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32,
                  u32, u32, C.c_void_p, u32, f32]),
    "qw_gpu_qk_norm_rope_cache_bf16": (
        C.c_int, [c_gpu] + [c_tensor] * 9 + [u32, u32, u32, u32, u32, f32]),
    "qw_gpu_attn_block_causal_bf16": (
        C.c_int, [c_gpu, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32, u32, u32, u32,
                  C.c_void_p, u32, f32]),
    "qw_gpu_device": (C.c_int, [c_gpu]),
    "qw_gpu_tensor_device_ptr": (C.c_void_p, [c_tensor]),
    "qw_gpu_stream": (C.c_void_p, [c_gpu]),
    "qw_gpu_host_alloc": (C.c_void_p, [size_t]),
    "qw_gpu_host_free": (None, [C.c_void_p]),
    "qw_gpu_tensor_read_async": (C.c_int, [c_gpu, c_tensor, C.c_void_p, size_t]),
    "qw_gpu_fence": (C.c_int, [c_gpu, C.c_int, C.c_int]),
    "qw_gpu_tensor_write_lane": (C.c_int, [c_gpu, c_tensor, C.c_void_p, size_t, C.c_int]),
    "qw_gpu_tensor_read_lane": (C.c_int, [c_gpu, c_tensor, C.c_void_p, size_t, C.c_int]),
    "qw_gpu_set_attention_kernel": (C.c_int, [c_gpu, C.c_char_p]),
    "qw_gpu_kernel_launches": (C.c_uint64, [c_gpu]),
    "qw_gpu_debug_attention_waits": (C.c_int, [c_gpu, C.c_longlong, C.c_int]),
    "qw_gpu_graph_begin": (C.c_int, [c_gpu]),
    "qw_gpu_graph_end": (C.c_void_p, [c_gpu]),
    "qw_gpu_graph_launch": (C.c_int, [c_gpu, C.c_void_p]),
    "qw_gpu_graph_free": (None, [C.c_void_p]),
    "qw_gpu_group_new_id": (C.c_int, [C.c_void_p, C.c_char_p, size_t]),
    "qw_gpu_group_join": (C.c_void_p, [c_gpu, C.c_void_p, C.c_int, C.c_int, C.c_char_p, size_t]),
    "qw_gpu_group_free": (None, [C.c_void_p]),
    "qw_gpu_group_rank": (C.c_int, [C.c_void_p]),
    "qw_gpu_group_world": (C.c_int, [C.c_void_p]),
    "qw_gpu_group_all_gather_heads_bf16": (C.c_int, [C.c_void_p, c_tensor, c_tensor, u32, u32, u32]),
    "qw_gpu_group_bind_output": (C.c_int, [C.c_void_p, c_tensor]),
    "qw_gpu_group_barrier": (C.c_int, [C.c_void_p]),
    "qw_gpu_group_wait_output": (C.c_int, [C.c_void_p, c_tensor]),
    "qw_gpu_group_attn_block_causal_bf16": (
        C.c_int, [C.c_void_p, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, c_tensor, u32, u32,
                  u32, u32, u32, C.c_void_p, u32, f32]),
    "qw_gpu_group_set_batch_groups": (C.c_int, [C.c_void_p, C.c_int]),
    "qw_gpu_group_batch_index": (C.c_int, [C.c_void_p]),
    "qw_gpu_group_head_index": (C.c_int, [C.c_void_p]),
    "qw_gpu_group_head_groups": (C.c_int, [C.c_void_p]),
    "qw_dit_prefix_limits": (None, [C.POINTER(Segment), u32, C.c_void_p]),
    "qw_pipe_rope_tables": (
        C.c_int, [c_gpu, u32, u32, u32, C.POINTER(c_tensor), C.POINTER(c_tensor), C.c_char_p, size_t]),
    "qw_pipe_rope_tables_blocks": (
        C.c_int, [c_gpu, C.c_void_p, C.c_void_p, C.c_void_p, u32, C.POINTER(c_tensor),
                  C.POINTER(c_tensor), C.c_char_p, size_t]),
    "qw_rope_tables_host": (u32, [u32, u32, u32, C.c_void_p, C.c_void_p]),
    "qw_rope_tables_blocks_host": (u32, [C.c_void_p, C.c_void_p, C.c_void_p, u32, C.c_void_p, C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it is missing (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C qwen_metal_b200/csrc` "
                "(or __graft_entry__.build()); there is no fallback implementation")
        lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def exported_names():
    return sorted(_SIGNATURES)


def _ptr(array: np.ndarray):
    return array.ctypes.data_as(C.c_void_p)


class GpuError(RuntimeError):
    pass


class Gpu:
    """A context (h3_gpu) with numpy-friendly helpers around the raw ABI."""

    def __init__(self, device: int | None = None):
        self.lib = load()
        err = C.create_string_buffer(512)
        if device is None:
            self.handle = self.lib.h3_gpu_create(b"h3_shaders.metal", err, len(err))
        else:
            self.handle = self.lib.qw_gpu_create_on_device(device, err, len(err))
        if not self.handle:
            raise GpuError(err.value.decode())
        self._tensors = []

    def close(self):
        if self.handle:
            for t in self._tensors:
                self.lib.h3_gpu_tensor_free(t)
            self._tensors = []
            self.lib.h3_gpu_free(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def error(self) -> str:
        return self.lib.h3_gpu_error(self.handle).decode()

    def check(self, ok, what="op"):
        if not ok:
            raise GpuError(f"{what}: {self.error()}")

    # -- tensors -----------------------------------------------------------
    def _track(self, t, what):
        if not t:
            raise GpuError(f"{what}: allocation failed: {self.error()}")
        self._tensors.append(t)
        return t

    def bf16(self, array: np.ndarray):
        a = np.ascontiguousarray(array, dtype=np.uint16)
        return self._track(self.lib.h3_gpu_tensor_from_bf16(self.handle, _ptr(a), a.size), "bf16")

    def f32(self, array: np.ndarray):
        a = np.ascontiguousarray(array, dtype=np.float32)
        return self._track(self.lib.h3_gpu_tensor_from_f32(self.handle, _ptr(a), a.size), "f32")

    def u32(self, array: np.ndarray):
        a = np.ascontiguousarray(array, dtype=np.uint32)
        return self._track(self.lib.h3_gpu_tensor_from_u32(self.handle, _ptr(a), a.size), "u32")

    def new_bf16(self, elements: int):
        return self._track(self.lib.h3_gpu_tensor_new_bf16(self.handle, elements), "new_bf16")

    def new_f32(self, elements: int):
        return self._track(self.lib.h3_gpu_tensor_new_f32(self.handle, elements), "new_f32")

    def free(self, tensor):
        self._tensors.remove(tensor)
        self.lib.h3_gpu_tensor_free(tensor)

    def read_bf16(self, tensor, elements: int) -> np.ndarray:
        out = np.empty(elements, dtype=np.uint16)
        self.check(self.lib.h3_gpu_tensor_read_bf16(tensor, _ptr(out), elements), "read_bf16")
        return out

    def read_f32(self, tensor, elements: int) -> np.ndarray:
        out = np.empty(elements, dtype=np.float32)
        self.check(self.lib.h3_gpu_tensor_read_f32(tensor, _ptr(out), elements), "read_f32")
        return out

    def write_bf16(self, tensor, array: np.ndarray):
        a = np.ascontiguousarray(array, dtype=np.uint16)
        self.check(self.lib.h3_gpu_tensor_write_bf16(tensor, _ptr(a), a.size), "write_bf16")

    # -- chain ---------------------------------------------------------------
    def begin(self):
        self.check(self.lib.h3_gpu_begin(self.handle), "begin")

    def submit(self):
        self.check(self.lib.h3_gpu_submit(self.handle), "submit")

    def stats(self) -> Stats:
        s = Stats()
        self.lib.h3_gpu_get_stats(self.handle, C.byref(s))
        return s


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even by the integer trick every path of the reference
    uses (h3_shaders.metal:15-19)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = bits + 0x7FFF + ((bits >> 16) & 1)
    return ((bits >> 16) & 0xFFFF).astype(np.uint16)


def prefix_limits(segments) -> np.ndarray:
    """qw_dit_prefix_limits through the library; segments = [(rows, is_image), ...]."""
    lib = load()
    arr = (Segment * len(segments))(*[Segment(r, int(i), 0) for r, i in segments])
    total = sum(r for r, _ in segments)
    out = np.zeros(total, dtype=np.uint32)
    lib.qw_dit_prefix_limits(arr, len(segments), _ptr(out))
    return out


def rope_tables(text_rows: int, gh: int, gw: int):
    lib = load()
    rows = text_rows + gh * gw
    cos = np.empty((rows, 64), dtype=np.float32)
    sin = np.empty((rows, 64), dtype=np.float32)
    got = lib.qw_rope_tables_host(text_rows, gh, gw, _ptr(cos), _ptr(sin))
    assert got == rows
    return cos, sin


def rope_tables_blocks(block_h, block_w, text_before):
    lib = load()
    bh = np.asarray(block_h, dtype=np.uint32)
    bw = np.asarray(block_w, dtype=np.uint32)
    tb = np.asarray(text_before, dtype=np.uint32)
    rows = int((tb + bh * bw).sum())
    cos = np.empty((rows, 64), dtype=np.float32)
    sin = np.empty((rows, 64), dtype=np.float32)
    got = lib.qw_rope_tables_blocks_host(_ptr(bh), _ptr(bw), _ptr(tb), len(bh), _ptr(cos), _ptr(sin))
    assert got == rows
    return cos, sin
