"""B200-native implementation of the Qwen-Image DiT attention hot path
(per-head QK RMSNorm -> 3-axis RoPE -> block-causal SDPA) behind the C ABI of
include/h3_gpu.h, include/qwen_gpu_ext.h and include/qwen_attn_host.h.

The product is the shared library under qwen_metal_b200/lib/ built from
qwen_metal_b200/csrc/; the Python modules here are the ctypes stub (abi) and the
workload definitions (workloads) that tests and the benchmark drive it with.
"""
from . import abi  # noqa: F401
