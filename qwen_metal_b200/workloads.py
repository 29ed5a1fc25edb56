"""The attention-path workloads: token layouts, seeded synthetic inputs and the
per-layer op sequence (reference qwen_dit.m:1273-1440) driven through the C ABI.

Config numbering follows the benchmark definition:
  0  the reference's own known-answer test (tests/test_prefix_kernel.c)
  1  256^2 image, text 64 + 16x16 latent tokens, SDPA only
  2  512^2 turbo single layer with the QK-norm + RoPE prologue
  3  1024^2 with classifier-free guidance: batch 2, text 200 / 32 padded to 256
  4  edit path: text 256 + condition image 64x64 + target image 64x64
  5  2048^2 with guidance, batch 2, text 512 + 128x128 latent tokens
"""
from __future__ import annotations

import dataclasses
import math
import os

import numpy as np

from . import abi

HEAD_DIM = 128
SCALE = 1.0 / math.sqrt(128.0)  # reference qwen_dit.m:19
EPS = 1e-6


@dataclasses.dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    heads: int
    runs: tuple            # ((rows, is_image), ...) of ONE batch item, padded text included
    grids: tuple           # ((gh, gw), ...) one per image run
    text_len: tuple = ()   # real text length per batch item (key padding) or ()
    text_pad: int = 0
    prologue: bool = True
    layers: int = 1
    text_bidirectional: bool = False

    @property
    def rows(self) -> int:
        return sum(r for r, _ in self.runs)

    def limits(self) -> np.ndarray:
        """Per-row key limits (integer, bit-exact contract) via the library's
        qw_dit_prefix_limits; text rows are token-causal as in the reference
        unless text_bidirectional asks for the run end instead."""
        lim = abi.prefix_limits(list(self.runs))
        if self.text_bidirectional:
            start = 0
            for rows, is_image in self.runs:
                if not is_image:
                    lim[start:start + rows] = start + rows
                start += rows
        return lim

    def rope_tables(self):
        """Joint 3-axis tables for one batch item (shared by the batch)."""
        text_before, bh, bw = [], [], []
        pending_text = 0
        grids = list(self.grids)
        for rows, is_image in self.runs:
            if is_image:
                gh, gw = grids.pop(0)
                assert gh * gw == rows
                text_before.append(pending_text)
                bh.append(gh)
                bw.append(gw)
                pending_text = 0
            else:
                pending_text += rows
        assert pending_text == 0, "the joint layout ends with an image run"
        return abi.rope_tables_blocks(bh, bw, text_before)

    def visible_pairs(self) -> int:
        """Sum over batch items and rows of the visible key count (one head)."""
        lim = self.limits().astype(np.int64)
        total = 0
        for b in range(self.batch):
            vis = lim.copy()
            if self.text_pad:
                tl = self.text_len[b]
                lo = np.minimum(tl, lim)
                hi = np.minimum(self.text_pad, lim)
                vis = lim - (hi - lo)
                vis[tl:self.text_pad] = 0
            total += int(vis.sum())
        return total

    def flops_per_layer(self) -> float:
        """Mask-aware FLOPs: 4 * D * H * sum(visible) (QK^T + PV, 2 flop/MAC;
        same convention as the reference's tests/bench_sdpa.c:162-164)."""
        return 4.0 * HEAD_DIM * self.heads * self.visible_pairs()

    def prologue_bytes_per_layer(self) -> float:
        elems = self.batch * self.rows * self.heads * HEAD_DIM
        return 2 * elems * 2 * 2 + 2 * self.rows * 64 * 4

    def attention_min_bytes_per_layer(self) -> float:
        elems = self.batch * self.rows * self.heads * HEAD_DIM
        return 4 * elems * 2


def workload(index: int, heads: int = 24) -> Workload:
    if index == 1:
        return Workload("cfg1 256^2 SDPA parity", 1, heads, ((64, 0), (256, 1)), ((16, 16),),
                        prologue=False)
    if index == 2:
        return Workload("cfg2 512^2 turbo layer", 1, heads, ((128, 0), (1024, 1)), ((32, 32),))
    if index == 3:
        return Workload("cfg3 1024^2 CFG batch 2", 2, heads, ((256, 0), (4096, 1)), ((64, 64),),
                        text_len=(200, 32), text_pad=256, layers=32)
    if index == 4:
        return Workload("cfg4 edit causal_condition", 1, heads,
                        ((256, 0), (4096, 1), (4096, 1)), ((64, 64), (64, 64)), layers=32)
    if index == 5:
        return Workload("cfg5 2048^2 CFG batch 2", 2, heads, ((512, 0), (16384, 1)),
                        ((128, 128),), text_len=(512, 512), text_pad=512, layers=32)
    raise ValueError(f"no workload {index}")


def normal_bf16(rng: np.random.Generator, shape, mean=0.0, std=1.0) -> np.ndarray:
    """Seeded N(mean, std) values rounded to bf16 (returned as uint16 bits)."""
    values = rng.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)
    return abi.f32_to_bf16(values)


def layer_inputs(w: Workload, layer: int, base_seed: int = 20261028):
    """q, k, v [batch, rows, heads, 128] bf16 bits and the two norm weights for
    one seeded layer; identical bytes go to the GPU and to the CPU oracle."""
    rng = np.random.default_rng([base_seed, layer, w.batch, w.rows, w.heads])
    shape = (w.batch, w.rows, w.heads, HEAD_DIM)
    q = normal_bf16(rng, shape)
    k = normal_bf16(rng, shape)
    v = normal_bf16(rng, shape)
    wq = normal_bf16(rng, (HEAD_DIM,), 1.0, 0.1)
    wk = normal_bf16(rng, (HEAD_DIM,), 1.0, 0.1)
    return q, k, v, wq, wk


class LayerRunner:
    """Device-resident state of one workload and the per-layer op sequence."""

    def __init__(self, gpu: abi.Gpu, w: Workload, heads_local: int | None = None,
                 bounded: bool | None = None, batch_items: tuple | None = None):
        """heads_local / batch_items = (first, count): this rank's share when the
        heads and the batch items are sharded over several GPUs."""
        self.gpu, self.w = gpu, w
        self.heads = heads_local or w.heads
        self.batch0, self.batch = batch_items or (0, w.batch)
        # With the QK-norm in front, the prologue also leaves the norm bounds of its
        # outputs on the device and the attention kernel runs its fixed-exponent
        # softmax; QW_SOFTMAX=max (or bounded=False) keeps the running-maximum path.
        if bounded is None:
            bounded = os.environ.get("QW_SOFTMAX", "bounded") != "max"
        self.bounded = bool(bounded and w.prologue)
        self.bound = gpu.new_f32(2) if self.bounded else None
        n = self.batch * w.rows * self.heads * HEAD_DIM
        self.n = n
        self.limits_host = w.limits()
        self.limits = gpu.u32(self.limits_host)
        if w.prologue:
            cos, sin = w.rope_tables()
            self.cos, self.sin = gpu.f32(cos), gpu.f32(sin)
        self.text_len = (np.asarray(w.text_len[self.batch0:self.batch0 + self.batch],
                                    dtype=np.uint32) if w.text_pad else None)
        self.out = gpu.new_bf16(n)

    def enqueue(self, q, k, v, wq=None, wk=None, out=None, q_work=None, k_work=None,
                group=None, full=None):
        """One layer: [fused QK-norm + RoPE] then block-causal attention.  With
        q_work/k_work the prologue writes there and leaves q, k untouched.  With a
        multi-GPU group and a bound `full` output the kernel writes this rank's head
        columns of `full` and the group's push kernel copies them to the peers."""
        g, w, lib = self.gpu, self.w, self.gpu.lib
        batch = self.batch
        out = out or self.out
        if w.prologue:
            qo, ko = (q_work or q), (k_work or k)
            if self.bounded:
                g.check(lib.qw_gpu_qk_norm_rope_bound_bf16(
                    g.handle, qo, ko, q, k, wq, wk, self.cos, self.sin, self.bound, batch,
                    w.rows, self.heads, HEAD_DIM, EPS), "qk_norm_rope_bound")
            else:
                g.check(lib.qw_gpu_qk_norm_rope_out_bf16(g.handle, qo, ko, q, k, wq, wk, self.cos,
                                                         self.sin, batch, w.rows, self.heads,
                                                         HEAD_DIM, EPS),
                        "qk_norm_rope")
            q, k = qo, ko
        tl = abi._ptr(self.text_len) if self.text_len is not None else None
        if group is not None:
            g.check(lib.qw_gpu_group_attn_block_causal_bf16(
                group, full, q, k, v, self.limits, self.bound if self.bounded else None, batch,
                w.rows, self.heads, self.heads, HEAD_DIM, tl, w.text_pad, SCALE),
                "group_attn_block_causal")
            return full
        if self.bounded:
            g.check(lib.qw_gpu_attn_block_causal_bounded_bf16(
                g.handle, out, q, k, v, self.limits, self.bound, batch, w.rows, self.heads,
                self.heads, HEAD_DIM, tl, w.text_pad, SCALE), "attn_block_causal_bounded")
            return out
        g.check(lib.qw_gpu_attn_block_causal_bf16(g.handle, out, q, k, v, self.limits, batch,
                                                  w.rows, self.heads, self.heads, HEAD_DIM, tl,
                                                  w.text_pad, SCALE),
                "attn_block_causal")
        return out
