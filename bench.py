#!/usr/bin/env python3
"""Benchmark of the DiT attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload 3]

A step is one 32-layer attention pass (per layer: fused QK-norm + RoPE, then
block-causal attention) over seeded synthetic inputs of the 1024^2 CFG workload
(batch 2, text 200 / 32 padded to 256, 4096 image tokens, 24 heads x 128).
With N > 1 (launched by torch.distributed.run, one rank per GPU) the ranks form
batch groups x head groups: the two guidance branches go to different ranks
first (they never exchange anything), then the heads are sharded and every
layer's [rows, heads*128] output is gathered inside a batch group by the
library's own push kernel over NVLink; the total work is fixed (strong scaling).

Prints ONE JSON line: whole-job mask-aware TFLOP/s (`value`, inputs resident in
HBM), the parity of what the timed step wrote against the CPU oracle on every
rank (`parity`; the run exits non-zero on a miss), the same metric end to end
from pinned HOST buffers through the C ABI (`e2e`), the dominant kernel's
roofline, the same for the largest configuration (`sweep_cfg5`), the CPU oracle
timed beside it (`cpu_baseline`) and the clocks seen during the timed region.

--impl reference times the CPU implementation of the path (the oracle port of
the reference's tests/test_prefix_kernel.c loop plus its scalar norm / RoPE
arithmetic, OpenMP over rows) on the host cores for the same metric; it loads
nothing of the product library.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

NOMINAL_BF16_TFLOPS = 2250.0
# (workload, GPUs) -> DRAM bytes one launch moved under ncu; see profiles/.
NCU_DRAM_BYTES = {
    (3, 1): {"attention": 193.9e6, "prologue": 172.5e6,
             "source": "profiles/attention_sm100_cfg3.txt, profiles/prologue_cfg3.txt"},
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d["bf16_tflops_sustained"]),
                "hbm": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the GPU runs the timed work
    (read only).  The sampler is started early and the samples are filtered by the
    host-clock windows in which timed work was in flight, so that a timed region
    shorter than the sampling period still gets its samples."""
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.path = device, None, f"/tmp/qw_clocks_{os.getpid()}.csv"
        self.windows = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.device)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
            return
        deadline = time.time() + 3.0  # first sample = the tool is up
        while time.time() < deadline and os.path.getsize(self.path) == 0:
            time.sleep(0.02)

    def window(self, t0, t1):
        self.windows.append((t0, t1))

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        self.proc.wait()
        import datetime
        inside, nearby = [], []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sample = (float(parts[2]), float(parts[3]),
                          [n for n, flag in zip(names, parts[6:10]) if flag.lower().startswith("active")])
            except ValueError:
                continue
            if any(t0 - 0.01 <= stamp <= t1 + 0.01 for t0, t1 in self.windows):
                inside.append(sample)
            elif any(t0 - 0.01 <= stamp <= t1 + 0.12 for t0, t1 in self.windows):
                nearby.append(sample)
        os.unlink(self.path)
        used = inside or nearby
        reasons = sorted({r for s_ in used for r in s_[2]})
        return {"sm_mhz": statistics.median([s_[0] for s_ in used]) if used else None,
                "sm_max_mhz": max(s_[1] for s_ in used) if used else None,
                "samples": len(used), "reasons": reasons,
                "sampled": "during the timed step and the per-kernel loops" if inside else
                           "within 0.12 s after the timed work (none fell inside it)"}


def oracle_limits(O, w):
    """Per-row key limits of the workload from the ORACLE's restatement of
    qw_dit_prefix_limits (the CPU legs load nothing of the product library)."""
    lim = O.prefix_limits(list(w.runs))
    if w.text_bidirectional:
        start = 0
        for rows, is_image in w.runs:
            if not is_image:
                lim[start:start + rows] = start + rows
            start += rows
    return lim


def oracle_rope_tables(O, w):
    text_before, bh, bw, pending, grids = [], [], [], 0, list(w.grids)
    for rows, is_image in w.runs:
        if is_image:
            gh, gw = grids.pop(0)
            text_before.append(pending), bh.append(gh), bw.append(gw)
            pending = 0
        else:
            pending += rows
    return O.rope_tables_blocks(bh, bw, text_before)


def oracle_flops_per_layer(O, w):
    tl = np.asarray(w.text_len, np.uint32) if w.text_pad else None
    pairs = O.visible_pairs(oracle_limits(O, w), w.batch, w.rows, w.rows, tl, w.text_pad)
    return 4.0 * 128 * w.heads * pairs


def oracle_prologue(O, w, q, k, wq, wk, cos, sin):
    from qwen_metal_b200 import workloads
    batch = q.shape[0]
    qn = O.head_rms_norm(q, wq, batch * w.rows, q.shape[2], workloads.EPS)
    kn = O.head_rms_norm(k, wk, batch * w.rows, k.shape[2], workloads.EPS)
    for b in range(batch):
        qn[b], kn[b] = O.qk_rope(qn[b], kn[b], cos, sin, w.rows, q.shape[2])
    return qn, kn


def cpu_sample(w, budget_s, chunk_rows=256, seed=17):
    """Time the CPU oracle on a bounded row sample of layer 0 of the workload:
    prologue on the whole layer once (it is cheap), then SDPA on seeded random
    query rows, all heads, in chunks until the budget is spent.  Returns
    (TFLOP/s over the SDPA sample, description, threads).  Everything here comes
    from the oracle; the product library is not touched."""
    import oracle_lib as O
    from qwen_metal_b200 import workloads
    O.use_all_cores()  # a launcher may have exported OMP_NUM_THREADS=1 to every rank
    q, k, v, wq, wk = workloads.layer_inputs(w, 0)
    cos, sin = oracle_rope_tables(O, w)
    t0 = time.perf_counter()
    qn, kn = oracle_prologue(O, w, q, k, wq, wk, cos, sin)
    t_prologue = time.perf_counter() - t0
    tl = np.asarray(w.text_len, np.uint32) if w.text_pad else None
    limits = oracle_limits(O, w)
    rng = np.random.default_rng(seed)
    done_rows, pairs, elapsed = 0, 0, 0.0
    while elapsed < budget_s:
        rows = rng.integers(0, w.batch * w.rows, chunk_rows).astype(np.uint32)
        t0 = time.perf_counter()
        _, visible = O.sdpa(qn, kn, v, limits, w.batch, w.rows, w.rows, w.heads, w.heads,
                            workloads.SCALE, tl, w.text_pad, rows)
        elapsed += time.perf_counter() - t0
        pairs += visible
        done_rows += chunk_rows
    flops = 4.0 * 128 * w.heads * pairs
    # charge the sample its share of the (whole-layer) prologue
    share = done_rows / float(w.batch * w.rows)
    tflops = flops / (elapsed + t_prologue * share) / 1e12
    sample = (f"{done_rows} seeded random query rows of layer 0 (all {w.heads} heads, "
              f"{pairs} visible pairs per head) in {elapsed:.1f} s; norm+RoPE of the layer "
              f"{t_prologue:.2f} s charged pro rata")
    return tflops, sample, O.threads()


def workload_config(w, **extra):
    """The `config` object both arms print (same keys, so the two lines compare)."""
    config = {"workload": w.name, "batch": w.batch, "rows": w.rows, "heads": w.heads,
              "head_dim": 128, "layers": w.layers, "text_len": list(w.text_len),
              "text_pad": w.text_pad}
    config.update(extra)
    return config


def run_reference(args):
    """The CPU implementation of the path on this box's host cores: the oracle port
    (the reference's CPU SDPA exists only inline in its test's main(), fixed at 149
    rows).  Loads oracle/ only: limits, tables and FLOP counts come from the oracle."""
    import oracle_lib as O
    from qwen_metal_b200 import workloads
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = workloads.workload(args.workload)
    steps = max(args.steps, 1)
    per_step = max(2.0, min(20.0, 120.0 / (steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_sample(w, min(per_step, 2.0))
    values, sample, threads = [], "", 1
    t0 = time.perf_counter()
    for _ in range(steps):
        v, sample, threads = cpu_sample(w, per_step)
        values.append(v)
    wall = time.perf_counter() - t0
    value = float(np.mean(values))
    layer_s = oracle_flops_per_layer(O, w) / (value * 1e12)
    line = {
        "impl": "reference", "metric": "block_causal_attn_tflops", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": layer_s * w.layers * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(
            w, parallelism="host cores (OpenMP over query rows)",
            l2="not applicable (CPU)",
            step="a time-bounded row sample of one layer; ms_per_step is extrapolated from it "
                 "to 32 layers x all rows"),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"each step: {sample}"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "wall_s": wall,
    }
    print(json.dumps(line), flush=True)


def parity_rows(w, count, seed):
    """Query rows of ONE batch item worth checking: every run / padding boundary
    +- 3, first and last rows, plus `count` seeded random rows."""
    edges = {0, w.rows - 1}
    start = 0
    for rows, _ in w.runs:
        for e in (start, start + rows):
            edges.update(range(max(0, e - 3), min(w.rows, e + 3)))
        start += rows
    for tl in w.text_len:
        edges.update(range(max(0, tl - 3), min(w.rows, tl + 3)))
    if w.text_pad:
        edges.update(range(max(0, w.text_pad - 3), min(w.rows, w.text_pad + 3)))
    rng = np.random.default_rng(seed)
    return sorted(edges | set(int(r) for r in rng.integers(0, w.rows, count)))


def parity_of_layer(w, layer, base_layer, got_bits, b0, nb, random_rows=64):
    """Compare this rank's gathered output of one layer (bf16 bits, [nb, rows,
    ALL heads, 128]) with the CPU oracle on a row sample.  `base_layer` is the seed
    index the layer's inputs were generated from.  Returns the error sums."""
    import oracle_lib as O
    from qwen_metal_b200 import abi, workloads
    O.use_all_cores()
    q, k, v, wq, wk = workloads.layer_inputs(w, base_layer)
    q, k, v = (x[b0:b0 + nb] for x in (q, k, v))
    cos, sin = oracle_rope_tables(O, w)
    qn, kn = oracle_prologue(O, w, q, k, wq, wk, cos, sin)
    per_item = parity_rows(w, random_rows, seed=1000 + layer)
    rows = np.array([b * w.rows + r for b in range(nb) for r in per_item], np.uint32)
    tl = np.asarray(w.text_len[b0:b0 + nb], np.uint32) if w.text_pad else None
    ref, _ = O.sdpa(qn, kn, v, oracle_limits(O, w), nb, w.rows, w.rows, w.heads, w.heads,
                    workloads.SCALE, tl, w.text_pad, rows)
    got = abi.bf16_to_f32(np.asarray(got_bits)).reshape(nb * w.rows, w.heads, 128)[rows]
    want = ref.reshape(nb * w.rows, w.heads, 128)[rows].astype(np.float64)
    diff = np.abs(got.astype(np.float64) - want)
    return {"max_abs": float(diff.max()), "abs_sum": float(diff.sum()), "count": int(diff.size),
            "diff_sq": float((diff ** 2).sum()), "ref_sq": float((want ** 2).sum()),
            "rows": int(rows.size), "finite": bool(np.isfinite(got).all())}


MAX_ABS, MEAN_ABS, REL_L2 = 2e-2, 2e-3, 5e-3   # the gates of tests/test_gpu_parity.py


class Job:
    """One workload on this rank: resident inputs, the per-step op sequence, the
    captured graph, timing and the parity check of what the timed step wrote."""

    def __init__(self, ctx, index, layers=0, distinct_layers=0, gather="push", cfg_split=True):
        import dataclasses
        from qwen_metal_b200 import sharding, workloads
        self.ctx = ctx
        gpu, world, rank = ctx.gpu, ctx.world, ctx.rank
        w = workloads.workload(index)
        if layers:
            w = dataclasses.replace(w, layers=layers)
        self.w, self.index = w, index
        groups = sharding.default_batch_groups(world, w.batch) if cfg_split else 1
        _, self.head_index, self.head_groups, self.b0, self.nb = sharding.layout(
            rank, world, w.batch, groups)
        self.batch_groups = groups
        if w.heads % self.head_groups:
            sys.exit(f"{w.heads} heads do not shard over {self.head_groups} ranks")
        self.heads_local = w.heads // self.head_groups
        self.gather = "none" if self.head_groups == 1 else gather
        if self.gather == "nccl" and groups != 1:
            sys.exit("--gather nccl needs --no-cfg-split (the NCCL gather spans all ranks)")
        if ctx.group:
            gpu.check(gpu.lib.qw_gpu_group_set_batch_groups(ctx.group, groups), "set_batch_groups")
        self.runner = workloads.LayerRunner(gpu, w, self.heads_local, batch_items=(self.b0, self.nb))
        self.n_local = self.runner.n
        self.n_full = self.nb * w.rows * w.heads * 128
        # distinct seeded input sets; layer i uses set i % distinct
        self.distinct = min(distinct_layers or w.layers, w.layers)
        self.layers, self.host_layers = [], []
        for layer in range(self.distinct):
            q, k, v, wq, wk = workloads.layer_inputs(w, layer)
            sl = [sharding.shard(x, rank, world, groups) for x in (q, k, v)]
            self.layers.append(tuple(gpu.bf16(x) for x in sl) + (gpu.bf16(wq), gpu.bf16(wk)))
            if layer < ctx.args.e2e_layers:
                self.host_layers.append(sl)
        self.q_work, self.k_work = gpu.new_bf16(self.n_local), gpu.new_bf16(self.n_local)
        # outputs alternate between two buffers, so the last two layers of the timed
        # step are both there to be checked afterwards
        if self.gather == "none":
            self.outs = [gpu.new_bf16(self.n_local) for _ in range(2)]
        else:
            self.outs = [gpu.new_bf16(self.n_full) for _ in range(2)]
            self.out_local = gpu.new_bf16(self.n_local)
            if self.gather == "push":
                for t in self.outs:  # collective: maps every rank's buffers over NVLink
                    gpu.check(gpu.lib.qw_gpu_group_bind_output(ctx.group, t), "bind_output")
        self.graph = None

    def one_step(self):
        gpu, lib, ctx, w = self.ctx.gpu, self.ctx.gpu.lib, self.ctx, self.w
        for i in range(w.layers):
            qt, kt, vt, wqt, wkt = self.layers[i % self.distinct]
            out = self.outs[i & 1]
            if self.gather == "push":
                self.runner.enqueue(qt, kt, vt, wqt, wkt, q_work=self.q_work, k_work=self.k_work,
                                    group=ctx.group, full=out)
            elif self.gather == "nccl":
                self.runner.enqueue(qt, kt, vt, wqt, wkt, out=self.out_local, q_work=self.q_work,
                                    k_work=self.k_work)
                gpu.check(lib.qw_gpu_group_all_gather_heads_bf16(
                    ctx.group, out, self.out_local, self.nb * w.rows, self.heads_local, 128),
                    "all_gather")
            else:
                self.runner.enqueue(qt, kt, vt, wqt, wkt, out=out, q_work=self.q_work,
                                    k_work=self.k_work)

    def capture(self):
        gpu, lib = self.ctx.gpu, self.ctx.gpu.lib
        gpu.begin()
        gpu.check(lib.qw_gpu_graph_begin(gpu.handle), "graph begin")
        self.one_step()
        self.graph = lib.qw_gpu_graph_end(gpu.handle)
        if not self.graph:
            sys.exit("graph capture: " + gpu.error())
        gpu.submit()

    def step(self):
        if self.graph:
            gpu = self.ctx.gpu
            gpu.check(gpu.lib.qw_gpu_graph_launch(gpu.handle, self.graph), "graph launch")
        else:
            self.one_step()

    def parity(self):
        """Check the outputs the LAST timed step left behind (layers L-2 and L-1 sit in
        the two output buffers) on every rank against the oracle; reduce over ranks."""
        import torch
        import torch.distributed as dist
        ctx, w = self.ctx, self.w
        acc = {"max_abs": 0.0, "abs_sum": 0.0, "count": 0, "diff_sq": 0.0, "ref_sq": 0.0,
               "rows": 0, "finite": True}
        checked = []
        for layer in sorted({max(w.layers - 2, 0), w.layers - 1}):
            out = self.outs[layer & 1]
            if self.gather == "none":
                # this rank holds all heads of its batch items (no head sharding)
                bits = ctx.gpu.read_bf16(out, self.n_local)
            else:
                bits = ctx.gpu.read_bf16(out, self.n_full)
            r = parity_of_layer(w, layer, layer % self.distinct, bits, self.b0, self.nb)
            acc["max_abs"] = max(acc["max_abs"], r["max_abs"])
            acc["finite"] = acc["finite"] and r["finite"]
            for key in ("abs_sum", "count", "diff_sq", "ref_sq", "rows"):
                acc[key] += r[key]
            checked.append(layer)
        mean_abs = acc["abs_sum"] / max(acc["count"], 1)
        rel = (acc["diff_sq"] / max(acc["ref_sq"], 1e-30)) ** 0.5
        ok = acc["finite"] and acc["max_abs"] <= MAX_ABS and mean_abs <= MEAN_ABS and rel < REL_L2
        vals = [acc["max_abs"], mean_abs, rel, float(acc["rows"]), float(ok)]
        ranks_ok = int(ok)
        if ctx.world > 1:
            t = torch.tensor(vals, dtype=torch.float64, device="cuda")
            worst = t.clone()
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            total = t.clone()
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
            vals = [float(worst[0]), float(worst[1]), float(worst[2]), float(total[3]), 0.0]
            ranks_ok = int(round(float(total[4])))
        return {"max_abs": vals[0], "mean_abs": vals[1], "rel_l2": vals[2], "rows": int(vals[3]),
                "ranks_ok": ranks_ok, "ranks": ctx.world, "ok": ranks_ok == ctx.world,
                "layers_checked": checked, "heads_checked": w.heads,
                "gates": {"max_abs": MAX_ABS, "mean_abs": MEAN_ABS, "rel_l2": REL_L2},
                "what": "outputs left in the two output buffers by the last replay of the timed "
                        "step, read back on every rank (all head columns of the rank's batch "
                        "items), against the CPU oracle on run/padding boundaries +-3 and 64 "
                        "seeded random rows per item; worst rank reported"}

    def free(self):
        if self.graph:
            self.ctx.gpu.lib.qw_gpu_graph_free(self.graph)
            self.graph = None


class Context:
    """Process-wide state of the product arm: rank, GPU context, multi-GPU group."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        from qwen_metal_b200 import abi
        self.args = args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            sys.exit("--gpus N > 1 needs one rank per GPU: launch with torch.distributed.run")
        torch.cuda.set_device(self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.gpu = abi.Gpu(self.local)
        self.group = None
        lib = self.gpu.lib
        if self.world > 1:
            ident = torch.zeros(128, dtype=torch.uint8)
            if self.rank == 0:
                buf = np.zeros(128, np.uint8)
                err = abi.C.create_string_buffer(256)
                if not lib.qw_gpu_group_new_id(abi._ptr(buf), err, 256):
                    sys.exit("group id: " + err.value.decode())
                ident = torch.from_numpy(buf)
            ident = ident.cuda()
            dist.broadcast(ident, 0)
            buf = ident.cpu().numpy()
            err = abi.C.create_string_buffer(256)
            self.group = lib.qw_gpu_group_join(self.gpu.handle, abi._ptr(buf), self.rank,
                                               self.world, err, 256)
            if not self.group:
                sys.exit("group join: " + err.value.decode())

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, *values):
        import torch
        import torch.distributed as dist
        if self.world == 1:
            return list(values)
        t = torch.tensor(values, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def timed(self, fn, reps):
        """Device time of `reps` calls of fn (CUDA events on the context's stream,
        recorded by begin/submit, which joins the communication stream before the
        stop event), max over ranks, in seconds."""
        gpu = self.gpu
        self.barrier()
        before = gpu.stats().gpu_seconds
        gpu.begin()
        for _ in range(reps):
            fn()
        gpu.submit()
        seconds = gpu.stats().gpu_seconds - before
        self.barrier()
        return self.max_over_ranks(seconds)[0]

    def close(self):
        import torch.distributed as dist
        if self.group:
            self.gpu.lib.qw_gpu_group_free(self.group)
        self.gpu.close()
        if self.world > 1:
            dist.destroy_process_group()


def measure_job(ctx, job, steps, warmup, sampler=None):
    """Warm up, capture the step into a graph, time `steps` replays, check what
    the last replay wrote.  Returns the record the JSON line is built from."""
    gpu, lib, w, args = ctx.gpu, ctx.gpu.lib, job.w, ctx.args
    ctx.timed(job.one_step, max(warmup, 3))
    if args.graph:
        # one step (32 layers) is captured once and replayed: the host cost of ~100 op
        # enqueues per step would otherwise bound short layers at N > 1
        job.capture()
        ctx.timed(job.step, 1)
    launches_before = lib.qw_gpu_kernel_launches(gpu.handle)
    wall0 = time.time()
    seconds = ctx.timed(job.step, steps)
    if sampler:
        sampler.window(wall0, time.time())
    launches = lib.qw_gpu_kernel_launches(gpu.handle) - launches_before
    parity = job.parity()
    flops_step = w.flops_per_layer() * w.layers          # all heads, all items: whole job
    value = flops_step * steps / seconds / 1e12
    parallelism = f"{job.batch_groups} batch group(s) x {job.head_groups} head group(s)"
    if job.gather == "push":
        parallelism += (": each rank writes its head columns of its own full output, a push "
                        "kernel copies them to the peers of its batch group under the next layer")
    elif job.gather == "nccl":
        parallelism += ": NCCL all-gather + interleave per layer"
    elif ctx.world > 1:
        parallelism += ": each rank owns whole batch items, nothing to gather"
    return {
        "value": value, "ms_per_step": seconds / steps * 1e3, "launches": int(launches),
        "parity": parity,
        "config": workload_config(
            w, parallelism=parallelism,
            l2="inputs larger than L2: %d distinct layers x %.0f MB of q,k,v per GPU stream "
               "through each step" % (job.distinct, 3 * job.n_local * 2 / 1e6),
            step=f"{w.layers} layers x (fused QK-norm+RoPE, block-causal attention"
                 + (", head push" if job.gather == "push" else "") + ")"
                 + (", replayed from a captured graph" if job.graph else "")),
    }


def kernel_rooflines(ctx, job, steps, peaks):
    """Attention and prologue kernels alone, each in a loop of steps x layers
    launches on this rank's share of the workload (the same entry points and the
    same kernels the step runs).  A kernel timed alone in a loop of well under a
    second is held against the measured BURST bf16 peak."""
    from qwen_metal_b200 import abi, workloads
    gpu, lib, w, runner = ctx.gpu, ctx.gpu.lib, job.w, job.runner
    tl = abi._ptr(runner.text_len) if runner.text_len is not None else None
    out = job.out_local if job.gather != "none" else job.outs[0]
    nb, hl = job.nb, job.heads_local

    def attention_only():
        # every layer's own raw q, k (N(0,1) rows: norms of about sqrt(128), inside or
        # within a few percent of the bound the prologue left behind, which guards
        # against overflow by a factor 2^60)
        for i in range(w.layers):
            qt, kt, vt, _, _ = job.layers[i % job.distinct]
            if runner.bounded:
                gpu.check(lib.qw_gpu_attn_block_causal_bounded_bf16(
                    gpu.handle, out, qt, kt, vt, runner.limits, runner.bound, nb, w.rows, hl, hl,
                    128, tl, w.text_pad, workloads.SCALE), "attention")
            else:
                gpu.check(lib.qw_gpu_attn_block_causal_bf16(
                    gpu.handle, out, qt, kt, vt, runner.limits, nb, w.rows, hl, hl, 128, tl,
                    w.text_pad, workloads.SCALE), "attention")

    def prologue_only():
        for i in range(w.layers):
            qt, kt, vt, wqt, wkt = job.layers[i % job.distinct]
            if runner.bounded:
                gpu.check(lib.qw_gpu_qk_norm_rope_bound_bf16(
                    gpu.handle, job.q_work, job.k_work, qt, kt, wqt, wkt, runner.cos, runner.sin,
                    runner.bound, nb, w.rows, hl, 128, workloads.EPS), "prologue")
            else:
                gpu.check(lib.qw_gpu_qk_norm_rope_out_bf16(
                    gpu.handle, job.q_work, job.k_work, qt, kt, wqt, wkt, runner.cos, runner.sin,
                    nb, w.rows, hl, 128, workloads.EPS), "prologue")

    launches = steps * w.layers
    attn_s = ctx.timed(attention_only, steps) / launches
    prol_s = ctx.timed(prologue_only, steps) / launches
    # this rank's share of the mask-aware FLOPs: its batch items, its heads
    import dataclasses
    share = dataclasses.replace(w, batch=nb, heads=hl,
                                text_len=tuple(w.text_len[job.b0:job.b0 + nb]))
    flops_launch = share.flops_per_layer()
    flops_launch = ctx.max_over_ranks(flops_launch)[0]   # the heaviest rank sets the time
    attn_tflops = flops_launch / attn_s / 1e12
    prol_bytes = (2 * job.n_local * 2 * 2) + 2 * w.rows * 64 * 4
    traffic = NCU_DRAM_BYTES.get((job.index, ctx.world), {})
    return {
        "kernel": "qw_attn_sm100_kernel", "bound": "tensor", "achieved": attn_tflops,
        "peak": peaks["bf16"], "unit": "TFLOP/s", "frac": attn_tflops / peaks["bf16"],
        "traffic": traffic.get("attention"), "traffic_source": traffic.get("source"),
        "peak_source": f"{peaks['source']} burst cuBLAS bf16 (the kernel is timed alone in a "
                       f"{launches}-launch loop of {attn_s * launches:.2f} s); sustained "
                       f"{peaks['bf16_sustained']}",
        "frac_of_sustained": attn_tflops / peaks["bf16_sustained"],
        "frac_of_nominal_2250": attn_tflops / NOMINAL_BF16_TFLOPS,
        "launch_ms": attn_s * 1e3, "flops_per_launch": flops_launch,
        "softmax": "fixed reference exponent from the QK-norm bound" if runner.bounded
                   else "running maximum",
        "prologue": {"kernel": "qw_prologue_kernel", "bound": "hbm",
                     "achieved": prol_bytes / prol_s / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": prol_bytes / prol_s / 1e9 / peaks["hbm"], "launch_ms": prol_s * 1e3,
                     "bytes_per_launch": prol_bytes, "traffic": traffic.get("prologue")},
    }


def gather_record(ctx, job, steps, attention_ms):
    """The sharded layer without its prologue: attention + head push, in a loop;
    what the push adds to a layer beyond the attention kernel is the exposed part."""
    if job.gather != "push":
        return None
    from qwen_metal_b200 import abi, workloads
    gpu, lib, w, runner = ctx.gpu, ctx.gpu.lib, job.w, job.runner
    tl = abi._ptr(runner.text_len) if runner.text_len is not None else None

    def sharded_attention():
        for i in range(w.layers):
            qt, kt, vt, _, _ = job.layers[i % job.distinct]
            gpu.check(lib.qw_gpu_group_attn_block_causal_bf16(
                ctx.group, job.outs[i & 1], qt, kt, vt, runner.limits,
                runner.bound if runner.bounded else None, job.nb, w.rows, job.heads_local,
                job.heads_local, 128, tl, w.text_pad, workloads.SCALE), "sharded attention")

    layer_s = ctx.timed(sharded_attention, steps) / (steps * w.layers)
    slice_bytes = job.nb * w.rows * job.heads_local * 128 * 2
    form = ("copy engines (one strided copy per peer) between two flag kernels"
            if os.environ.get("QW_CUDA_GROUP_PUSH") == "ce" else "push kernel")
    return {"mode": form + " over peer-mapped memory (NVLink), flag hand-shake, no NCCL call",
            "peers": job.head_groups - 1,
            "nvlink_bytes_out_per_launch": slice_bytes * (job.head_groups - 1),
            "attention_plus_push_ms_per_layer": layer_s * 1e3,
            "attention_alone_ms": attention_ms,
            "exposed_ms_per_layer": max(layer_s * 1e3 - attention_ms, 0.0)}


def neighbour_rooflines(ctx, job, peaks):
    """The block's element-wise neighbours of the path (single GPU only): the AdaLN
    norm in front of the QKV projection and the gated residual behind the output
    projection, on [batch*rows, heads*128] activations of this workload."""
    from qwen_metal_b200 import workloads
    gpu, lib, w = ctx.gpu, ctx.gpu.lib, job.w
    rows_all, width = w.batch * w.rows, job.heads_local * 128
    rng = np.random.default_rng(7)
    modulation = gpu.bf16(workloads.normal_bf16(rng, (2, 4, width), 0.0, 0.5))
    row_map = gpu.u32((np.arange(rows_all) % w.rows < (w.text_pad or 0)).astype(np.uint32))
    acts = [job.layers[i % len(job.layers)][0] for i in range(4)]  # resident q tensors

    def norm_only():
        for x in acts:
            gpu.check(lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, job.q_work, x, modulation, row_map,
                                                     rows_all, width, 4, 0, 1e-6), "norm")

    def gate_only():
        for i, x in enumerate(acts):
            gpu.check(lib.h3_gpu_gate_bf16(gpu.handle, job.q_work, x, acts[(i + 1) % 4], modulation,
                                           row_map, rows_all, width, 4, 2), "gate")

    ctx.timed(norm_only, 2), ctx.timed(gate_only, 2)
    norm_s = ctx.timed(norm_only, 5) / 20
    gate_s = ctx.timed(gate_only, 5) / 20
    n = job.n_local
    gpu.free(modulation), gpu.free(row_map)
    # the projections either side of the path on this workload's activations:
    # [batch*rows, H*128] x three [H*128, H*128] weights, and the output projection
    wts = [gpu.bf16(workloads.normal_bf16(rng, (width, width), 0.0, width ** -0.5)) for _ in range(3)]
    outs = [gpu.new_bf16(rows_all * width) for _ in range(3)]
    x = acts[0]

    def qkv_only():
        gpu.check(lib.qw_gpu_qkv_bf16(gpu.handle, *outs, x, *wts, rows_all, width), "qkv")

    def qkv_fused():
        _, _, _, wqt, wkt = job.layers[0]
        gpu.check(lib.qw_gpu_qkv_norm_rope_bf16(gpu.handle, *outs, x, *wts, wqt, wkt, job.runner.cos,
                                                job.runner.sin, None, w.batch, w.rows, width, 1e-6),
                  "qkv fused")

    def out_proj():
        gpu.check(lib.h3_gpu_linear_bf16(gpu.handle, outs[0], x, wts[0], None, rows_all, width,
                                         width), "linear")

    gemms = {}
    for name, fn, mult in (("qkv_projection", qkv_only, 3), ("qkv_projection_norm_rope", qkv_fused, 3),
                           ("output_projection", out_proj, 1)):
        ctx.timed(fn, 2)
        s_ = ctx.timed(fn, 10) / 10
        flops = 2.0 * rows_all * width * width * mult
        gemms[name] = {"kernel": "qw_linear_sm100_kernel", "bound": "tensor",
                       "flops_per_launch": flops, "achieved": flops / s_ / 1e12, "unit": "TFLOP/s",
                       "peak": peaks["bf16"], "frac": flops / s_ / 1e12 / peaks["bf16"],
                       "launch_ms": s_ * 1e3, "shape": [rows_all, width, width * mult]}
    for t in wts + outs:
        gpu.free(t)
    return {
        **gemms,
        "layer_norm_mod": {"bound": "hbm", "bytes_per_launch": 2 * n * 2,
                           "achieved": 2 * n * 2 / norm_s / 1e9, "unit": "GB/s",
                           "frac": 2 * n * 2 / norm_s / 1e9 / peaks["hbm"],
                           "launch_ms": norm_s * 1e3},
        "gate": {"bound": "hbm", "bytes_per_launch": 3 * n * 2,
                 "achieved": 3 * n * 2 / gate_s / 1e9, "unit": "GB/s",
                 "frac": 3 * n * 2 / gate_s / 1e9 / peaks["hbm"], "launch_ms": gate_s * 1e3},
    }


def run_product(args):
    ctx = Context(args)
    gpu, lib, world, rank = ctx.gpu, ctx.gpu.lib, ctx.world, ctx.rank
    peaks = measured_peaks()
    job = Job(ctx, args.workload, layers=args.layers, distinct_layers=args.distinct_layers,
              gather=args.gather, cfg_split=args.cfg_split)
    w = job.w
    sampler = ClockSampler(ctx.local)
    if rank == 0:
        sampler.start()
    main = measure_job(ctx, job, args.steps, args.warmup, sampler)

    wall0 = time.time()
    roofline = kernel_rooflines(ctx, job, args.steps, peaks)
    gather = gather_record(ctx, job, args.steps, roofline["launch_ms"])
    sampler.window(wall0, time.time())
    clocks = sampler.stop() if rank == 0 else None
    if gather:
        roofline["gather"] = gather
    if world == 1:
        roofline["neighbours"] = neighbour_rooflines(ctx, job, peaks)

    e2e = run_e2e(ctx, job) if args.e2e else None

    sweep = None
    if args.sweep and args.workload != 5:
        # the largest configuration, full 32 layers, at this N (4 distinct seeded input
        # sets cycled over the layers: 2.5 GB, larger than L2)
        big = Job(ctx, 5, layers=args.layers, distinct_layers=4, gather=args.gather,
                  cfg_split=args.cfg_split)
        rec = measure_job(ctx, big, max(1, min(args.steps, 5)), 3)
        sweep = {"metric": "block_causal_attn_tflops", "value": rec["value"], "unit": "TFLOP/s",
                 "n_gpus": world, "steps": max(1, min(args.steps, 5)), "warmup": 3,
                 "ms_per_step": rec["ms_per_step"], "ms_per_32_layer_pass": rec["ms_per_step"],
                 "tflops_per_gpu": rec["value"] / world,
                 "pct_bf16_peak_measured_burst": 100 * rec["value"] / world / peaks["bf16"],
                 "scaling": "strong", "dtype": "bf16", "data": "synthetic",
                 "config": rec["config"], "gpu_launches": rec["launches"],
                 "parity": rec["parity"]}
        big.free()

    cpu = None
    if rank == 0 and not args.no_cpu:
        v, sample, threads = cpu_sample(w, args.cpu_seconds)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}

    ok = main["parity"]["ok"] and (sweep is None or sweep["parity"]["ok"])
    if rank == 0:
        value = main["value"]
        line = {
            "metric": "block_causal_attn_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": main["config"],
            "tflops_per_gpu": value / world,
            "pct_bf16_peak_measured_burst": 100 * value / world / peaks["bf16"],
            "pct_bf16_peak_measured_sustained": 100 * value / world / peaks["bf16_sustained"],
            "pct_bf16_peak_nominal": 100 * value / world / NOMINAL_BF16_TFLOPS,
            "ms_per_32_layer_pass": main["ms_per_step"],
            "gpu_launches": main["launches"], "parity": main["parity"], "roofline": roofline,
            "cpu_baseline": cpu, "clocks": clocks, "e2e": e2e, "sweep_cfg5": sweep,
        }
        print(json.dumps(line), flush=True)
    job.free()
    ctx.close()
    if not ok:
        sys.exit("parity check failed: " + json.dumps(main["parity"]))


def run_e2e(ctx, job):
    """Same metric through the C-ABI calls a host program makes: every layer's
    q, k, v (this rank's share) start in pinned HOST memory, the ops run, and the
    layer's output -- the full gathered [rows, H*128] of the rank's batch items --
    is read back to pinned host memory.  Host wall clock, max over ranks."""
    import ctypes as C
    args, gpu, w, runner, world = ctx.args, ctx.gpu, job.w, job.runner, ctx.world
    lib = gpu.lib
    n = job.n_local
    n_out = job.n_full if job.gather != "none" else n
    nl = len(job.host_layers)
    pinned = []
    for sl in job.host_layers:
        bufs = []
        for x in sl:
            p = lib.qw_gpu_host_alloc(n * 2)
            if not p:
                return {"value": None, "unit": "TFLOP/s", "error": "pinned allocation failed"}
            C.memmove(p, x.ctypes.data, n * 2)
            bufs.append(p)
        pinned.append(bufs)
    out_host = [lib.qw_gpu_host_alloc(n_out * 2) for _ in range(2)]
    sets = [tuple(gpu.new_bf16(n) for _ in range(3)) for _ in range(2)]
    UP, DOWN = 1, 2   # lanes beside the compute stream

    def step():
        # upload of layer i+1, compute of layer i and read-back of layer i-1 overlap:
        # two device input sets, two output buffers, three streams joined by fences
        def upload(i):
            for t, h in zip(sets[i & 1], pinned[i % nl]):
                gpu.check(lib.qw_gpu_tensor_write_lane(gpu.handle, t, h, n, UP), "upload")
        upload(0)
        for i in range(w.layers):
            gpu.check(lib.qw_gpu_fence(gpu.handle, UP, 0), "fence")        # layer i is here
            if i + 1 < w.layers:
                gpu.check(lib.qw_gpu_fence(gpu.handle, 0, UP), "fence")    # set (i+1)&1 was read
                upload(i + 1)
            gpu.check(lib.qw_gpu_fence(gpu.handle, DOWN, 0), "fence")      # out[i&1] was read back
            dq, dk, dv = sets[i & 1]
            _, _, _, wqt, wkt = job.layers[i % job.distinct]
            out = job.outs[i & 1]
            if job.gather == "push":
                runner.enqueue(dq, dk, dv, wqt, wkt, q_work=job.q_work, k_work=job.k_work,
                               group=ctx.group, full=out)
                gpu.check(lib.qw_gpu_group_wait_output(ctx.group, out), "wait_output")
            elif job.gather == "nccl":
                runner.enqueue(dq, dk, dv, wqt, wkt, out=job.out_local, q_work=job.q_work,
                               k_work=job.k_work)
                gpu.check(lib.qw_gpu_group_all_gather_heads_bf16(
                    ctx.group, out, job.out_local, job.nb * w.rows, job.heads_local, 128), "gather")
            else:
                runner.enqueue(dq, dk, dv, wqt, wkt, out=out, q_work=job.q_work, k_work=job.k_work)
            gpu.check(lib.qw_gpu_fence(gpu.handle, 0, DOWN), "fence")
            gpu.check(lib.qw_gpu_tensor_read_lane(gpu.handle, out, out_host[i & 1], n_out, DOWN),
                      "read")

    steps = max(1, min(args.steps, 5))
    gpu.begin(); step(); gpu.submit()
    ctx.barrier()
    before = gpu.stats().gpu_seconds
    t0 = time.perf_counter()
    gpu.begin()
    for _ in range(steps):
        step()
    gpu.submit()
    ctx.barrier()
    wall = time.perf_counter() - t0
    device_s = gpu.stats().gpu_seconds - before
    wall, device_s = ctx.max_over_ranks(wall, device_s)
    # the last layer's read-back equals what the device holds
    check = np.frombuffer(C.string_at(out_host[(w.layers - 1) & 1], 4096), np.uint16)
    same = bool(np.array_equal(check, gpu.read_bf16(job.outs[(w.layers - 1) & 1], 2048)))
    for bufs in pinned:
        for p in bufs:
            lib.qw_gpu_host_free(p)
    for p in out_host:
        lib.qw_gpu_host_free(p)
    for s_ in sets:
        for t in s_:
            gpu.free(t)
    flops = w.flops_per_layer() * w.layers * steps
    return {"value": flops / wall / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": 3 * n * 2 * w.layers * world,
            "d2h_bytes_per_step": n_out * 2 * w.layers * world,
            "ms_per_step": wall / steps * 1e3, "device_ms_per_step": device_s / steps * 1e3,
            "steps": steps, "readback_matches_device": same,
            "note": f"host wall clock around {steps} steps incl. submit, max over ranks; byte "
                    f"counts summed over the {world} rank(s); {nl} distinct pinned layer input "
                    "sets cycled over the layers; uploads, compute and read-backs overlap on "
                    "three streams (two device input sets, two output buffers)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", type=int, default=3, choices=[2, 3, 4, 5])
    ap.add_argument("--layers", type=int, default=0,
                    help="override the layer count (small captures under a profiler)")
    ap.add_argument("--distinct-layers", type=int, default=0,
                    help="generate only this many distinct seeded input sets and cycle them over "
                         "the layers (quick experiments; default: one per layer)")
    ap.add_argument("--gather", default="push", choices=["push", "nccl"],
                    help="head groups > 1: the library's push kernel over peer memory, or NCCL "
                         "all-gather + interleave (comparison; needs --no-cfg-split)")
    ap.add_argument("--no-cfg-split", dest="cfg_split", action="store_false",
                    help="shard heads only; by default the batch items (guidance branches) are "
                         "split across ranks first")
    ap.add_argument("--no-sweep", dest="sweep", action="store_false",
                    help="skip the cfg5 (2048^2, 32 layers) sub-record")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="enqueue every op of every step from the host instead of replaying a graph")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-e2e", dest="e2e", action="store_false")
    ap.add_argument("--e2e-layers", type=int, default=4,
                    help="distinct pinned host input sets kept for the end-to-end leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_product(args)


if __name__ == "__main__":
    main()
