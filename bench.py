#!/usr/bin/env python3
"""Benchmark of the DiT attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload 3]

A step is one 32-layer attention pass (per layer: fused QK-norm + RoPE, then
block-causal attention) over seeded synthetic inputs of the 1024^2 CFG workload
(batch 2, text 200 / 32 padded to 256, 4096 image tokens, 24 heads x 128).
With N > 1 (launched by torch.distributed.run, one rank per GPU) the heads are
sharded N ways and every layer's [rows, heads*128] output is all-gathered with
NCCL; the total work is fixed (strong scaling).

Prints ONE JSON line: whole-job mask-aware TFLOP/s (`value`, inputs resident in
HBM), the same metric end to end from pinned HOST buffers through the C ABI
(`e2e`), the dominant kernel's roofline, the CPU oracle timed beside it
(`cpu_baseline`) and the clocks seen during the timed region.

--impl reference times the CPU implementation of the path (the oracle port of
the reference's tests/test_prefix_kernel.c loop plus its scalar norm / RoPE
arithmetic, OpenMP over rows) on the host cores for the same metric.
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
    (3, 1): {"attention": 193.7e6, "prologue": 172.5e6,
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


def oracle_prologue(O, w, q, k, wq, wk, cos, sin):
    from qwen_metal_b200 import workloads
    rows = w.batch * w.rows
    qn = O.head_rms_norm(q, wq, rows, q.shape[2], workloads.EPS)
    kn = O.head_rms_norm(k, wk, rows, k.shape[2], workloads.EPS)
    for b in range(w.batch):
        qn[b], kn[b] = O.qk_rope(qn[b], kn[b], cos, sin, w.rows, q.shape[2])
    return qn, kn


def cpu_sample(w, budget_s, chunk_rows=256, seed=17):
    """Time the CPU oracle on a bounded row sample of layer 0 of the workload:
    prologue on the whole layer once (it is cheap), then SDPA on seeded random
    query rows, all heads, in chunks until the budget is spent.  Returns
    (TFLOP/s over the SDPA sample, description, threads)."""
    import oracle_lib as O
    from qwen_metal_b200 import workloads
    O.use_all_cores()  # a launcher may have exported OMP_NUM_THREADS=1 to every rank
    q, k, v, wq, wk = workloads.layer_inputs(w, 0)
    cos, sin = w.rope_tables()
    t0 = time.perf_counter()
    qn, kn = oracle_prologue(O, w, q, k, wq, wk, cos, sin)
    t_prologue = time.perf_counter() - t0
    tl = np.asarray(w.text_len, np.uint32) if w.text_pad else None
    limits = w.limits()
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


def run_reference(args):
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
    layer_s = w.flops_per_layer() / (value * 1e12)
    line = {
        "impl": "reference", "metric": "block_causal_attn_tflops", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": layer_s * w.layers * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "batch": w.batch, "rows": w.rows, "heads": w.heads,
                   "layers": w.layers, "note": "ms_per_step extrapolated from the row sample"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"each step: {sample}"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "wall_s": wall,
    }
    print(json.dumps(line), flush=True)


def run_product(args):
    import torch
    import torch.distributed as dist
    from qwen_metal_b200 import abi, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            sys.exit("--gpus N > 1 needs one rank per GPU: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    w = workloads.workload(args.workload)
    if args.layers:
        import dataclasses
        w = dataclasses.replace(w, layers=args.layers)
    if w.heads % world:
        sys.exit(f"{w.heads} heads do not shard over {world} ranks")
    heads_local = w.heads // world
    peaks = measured_peaks()
    gpu = abi.Gpu(local)
    lib = gpu.lib
    group = None
    if world > 1:
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = np.zeros(128, np.uint8)
            err = abi.C.create_string_buffer(256)
            if not lib.qw_gpu_group_new_id(abi._ptr(buf), err, 256):
                sys.exit("group id: " + err.value.decode())
            ident = torch.from_numpy(buf)
        ident = ident.cuda()
        dist.broadcast(ident, 0)
        buf = ident.cpu().numpy()
        err = abi.C.create_string_buffer(256)
        group = lib.qw_gpu_group_join(gpu.handle, abi._ptr(buf), rank, world, err, 256)
        if not group:
            sys.exit("group join: " + err.value.decode())

    # ---- inputs: 32 seeded layers, this rank's head slice, resident in HBM ----
    runner = workloads.LayerRunner(gpu, w, heads_local)
    n_local = runner.n
    layers = []
    host_layers = []
    h0 = rank * heads_local
    for layer in range(w.layers):
        q, k, v, wq, wk = workloads.layer_inputs(w, layer)
        sl = [np.ascontiguousarray(x[:, :, h0:h0 + heads_local]) for x in (q, k, v)]
        layers.append(tuple(gpu.bf16(x) for x in sl) + (gpu.bf16(wq), gpu.bf16(wk)))
        if args.e2e and layer < args.e2e_layers:
            host_layers.append(sl)
    q_work, k_work = gpu.new_bf16(n_local), gpu.new_bf16(n_local)
    out_local = gpu.new_bf16(n_local)
    rows_total = w.batch * w.rows
    fused = world > 1 and args.gather == "fused"
    out_full = [gpu.new_bf16(n_local * world) for _ in range(2)] if world > 1 else None
    if fused:
        for t in out_full:  # collective: maps every rank's buffers over the NVLink peer path
            gpu.check(lib.qw_gpu_group_bind_output(group, t), "bind_output")

    def one_step():
        for i, (qt, kt, vt, wqt, wkt) in enumerate(layers):
            if fused:
                # the kernel's epilogue stores this rank's heads into every rank's full
                # output, then the ranks meet at a barrier; two outputs alternate
                runner.enqueue(qt, kt, vt, wqt, wkt, q_work=q_work, k_work=k_work, group=group,
                               full=out_full[i & 1])
                continue
            runner.enqueue(qt, kt, vt, wqt, wkt, out=out_local, q_work=q_work, k_work=k_work)
            if group:
                gpu.check(lib.qw_gpu_group_all_gather_heads_bf16(group, out_full[i & 1], out_local,
                                                                 rows_total, heads_local, 128),
                          "all_gather")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, reps):
        """Device time of `reps` calls of fn (CUDA events on the context's stream,
        recorded by begin/submit), max over ranks, in seconds."""
        barrier()
        before = gpu.stats().gpu_seconds
        gpu.begin()
        for _ in range(reps):
            fn()
        gpu.submit()
        seconds = gpu.stats().gpu_seconds - before
        barrier()
        if world > 1:
            t = torch.tensor([seconds], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            seconds = float(t.item())
        return seconds

    timed(one_step, max(args.warmup, 3))
    # One step (32 layers) is captured once and replayed: the host cost of ~100 op
    # enqueues per step would otherwise bound short layers at N > 1.
    step = one_step
    graph = None
    if args.graph:
        gpu.begin()
        gpu.check(lib.qw_gpu_graph_begin(gpu.handle), "graph begin")
        one_step()
        graph = lib.qw_gpu_graph_end(gpu.handle)
        if not graph:
            sys.exit("graph capture: " + gpu.error())
        gpu.submit()

        def step():
            gpu.check(lib.qw_gpu_graph_launch(gpu.handle, graph), "graph launch")
        timed(step, 1)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches_before = lib.qw_gpu_kernel_launches(gpu.handle)
    wall0 = time.time()
    seconds = timed(step, args.steps)
    sampler.window(wall0, time.time())
    launches = lib.qw_gpu_kernel_launches(gpu.handle) - launches_before

    flops_step = w.flops_per_layer() * w.layers          # all heads, whole job
    value = flops_step * args.steps / seconds / 1e12
    ms_per_step = seconds / args.steps * 1e3

    # ---- per-kernel timing for the roofline (attention alone, prologue alone) ----
    tl = abi._ptr(runner.text_len) if runner.text_len is not None else None

    def attention_only():
        # the same entry point the step uses, on every layer's own raw q, k (N(0,1) rows:
        # norms of about sqrt(128), inside or within a few percent of the bound the
        # prologue left behind, which guards against overflow by a factor 2^60)
        for (qt, kt, vt, _, _) in layers:
            if runner.bounded:
                gpu.check(lib.qw_gpu_attn_block_causal_bounded_bf16(
                    gpu.handle, out_local, qt, kt, vt, runner.limits, runner.bound, w.batch,
                    w.rows, heads_local, heads_local, 128, tl, w.text_pad, workloads.SCALE),
                    "attention")
            else:
                gpu.check(lib.qw_gpu_attn_block_causal_bf16(
                    gpu.handle, out_local, qt, kt, vt, runner.limits, w.batch, w.rows,
                    heads_local, heads_local, 128, tl, w.text_pad, workloads.SCALE), "attention")

    def prologue_only():
        for (qt, kt, vt, wqt, wkt) in layers:
            if runner.bounded:
                gpu.check(lib.qw_gpu_qk_norm_rope_bound_bf16(
                    gpu.handle, q_work, k_work, qt, kt, wqt, wkt, runner.cos, runner.sin,
                    runner.bound, w.batch, w.rows, heads_local, 128, workloads.EPS), "prologue")
            else:
                gpu.check(lib.qw_gpu_qk_norm_rope_out_bf16(
                    gpu.handle, q_work, k_work, qt, kt, wqt, wkt, runner.cos, runner.sin, w.batch,
                    w.rows, heads_local, 128, workloads.EPS), "prologue")

    wall0 = time.time()
    attn_s = timed(attention_only, args.steps) / (args.steps * w.layers)
    prol_s = timed(prologue_only, args.steps) / (args.steps * w.layers)
    sampler.window(wall0, time.time())
    clocks = sampler.stop() if rank == 0 else None
    flops_launch = w.flops_per_layer() / world
    attn_tflops = flops_launch / attn_s / 1e12
    prol_bytes = (2 * n_local * 2 * 2) + 2 * w.rows * 64 * 4
    # DRAM bytes per launch from the committed ncu captures (dram__bytes_read.sum +
    # dram__bytes_write.sum), known for the single-GPU cfg3 launch only.
    traffic = NCU_DRAM_BYTES.get((args.workload, world), {})
    roofline = {
        "kernel": "qw_attn_sm100_kernel", "bound": "tensor", "achieved": attn_tflops,
        "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
        "frac": attn_tflops / peaks["bf16_sustained"], "traffic": traffic.get("attention"),
        "traffic_source": traffic.get("source"),
        "peak_source": f"{peaks['source']} sustained cuBLAS bf16 (kernel timed in a "
                       f"{args.steps * w.layers}-launch loop); burst {peaks['bf16']}",
        "launch_ms": attn_s * 1e3, "flops_per_launch": flops_launch,
        "frac_of_nominal_2250": attn_tflops / NOMINAL_BF16_TFLOPS,
        "prologue": {"kernel": "qw_prologue_kernel", "bound": "hbm",
                     "achieved": prol_bytes / prol_s / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": prol_bytes / prol_s / 1e9 / peaks["hbm"], "launch_ms": prol_s * 1e3,
                     "bytes_per_launch": prol_bytes, "traffic": traffic.get("prologue")},
    }

    # ---- the block's element-wise neighbours of the path (single GPU only): the
    # AdaLN norm in front of the QKV projection and the gated residual behind the
    # output projection, on [batch*rows, heads*128] activations of this workload ----
    if world == 1:
        rows_all, width = w.batch * w.rows, heads_local * 128
        rng = np.random.default_rng(7)
        modulation = gpu.bf16(workloads.normal_bf16(rng, (2, 4, width), 0.0, 0.5))
        row_map = gpu.u32((np.arange(rows_all) % w.rows < (w.text_pad or 0)).astype(np.uint32))
        acts = [layers[i % len(layers)][0] for i in range(4)]  # resident q tensors as activations

        def norm_only():
            for i, x in enumerate(acts):
                gpu.check(lib.qw_gpu_layer_norm_mod_bf16(gpu.handle, q_work, x, modulation, row_map,
                                                         rows_all, width, 4, 0, 1e-6), "norm")

        def gate_only():
            for i, x in enumerate(acts):
                gpu.check(lib.h3_gpu_gate_bf16(gpu.handle, q_work, x, acts[(i + 1) % 4], modulation,
                                               row_map, rows_all, width, 4, 2), "gate")

        timed(norm_only, 2), timed(gate_only, 2)
        norm_s = timed(norm_only, 5) / 20
        gate_s = timed(gate_only, 5) / 20
        roofline["neighbours"] = {
            "layer_norm_mod": {"bound": "hbm", "bytes_per_launch": 2 * n_local * 2,
                               "achieved": 2 * n_local * 2 / norm_s / 1e9, "unit": "GB/s",
                               "frac": 2 * n_local * 2 / norm_s / 1e9 / peaks["hbm"],
                               "launch_ms": norm_s * 1e3},
            "gate": {"bound": "hbm", "bytes_per_launch": 3 * n_local * 2,
                     "achieved": 3 * n_local * 2 / gate_s / 1e9, "unit": "GB/s",
                     "frac": 3 * n_local * 2 / gate_s / 1e9 / peaks["hbm"],
                     "launch_ms": gate_s * 1e3},
        }
        gpu.free(modulation), gpu.free(row_map)

    # ---- end to end from pinned host buffers through the C ABI (N = 1) ----
    e2e = None
    if args.e2e and (world == 1 or fused):
        e2e = run_e2e(args, gpu, w, runner, host_layers, layers, out_local,
                      group if fused else None, out_full, world, barrier)

    cpu = None
    if rank == 0 and not args.no_cpu:
        v, sample, threads = cpu_sample(w, args.cpu_seconds)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": "block_causal_attn_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w.name, "batch": w.batch, "rows": w.rows, "heads": w.heads,
                       "head_dim": 128, "layers": w.layers, "text_len": list(w.text_len),
                       "text_pad": w.text_pad,
                       "parallelism": f"heads/{world}" + (
                           "" if world == 1 else
                           " + fused peer-store gather in the attention epilogue + barrier"
                           if fused else " + NCCL all-gather + interleave per layer"),
                       "l2": "inputs larger than L2: 32 layers x %.0f MB of q,k,v stream through "
                             "each step" % (3 * n_local * 2 / 1e6),
                       "step": "32 layers x (fused QK-norm+RoPE, block-causal attention)"
                               + (", replayed from a captured graph" if graph else "")},
            "tflops_per_gpu": value / world,
            "pct_bf16_peak_measured_burst": 100 * value / world / peaks["bf16"],
            "pct_bf16_peak_nominal": 100 * value / world / NOMINAL_BF16_TFLOPS,
            "ms_per_32_layer_pass": ms_per_step,
            "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
            "clocks": clocks, "e2e": e2e,
        }
        print(json.dumps(line), flush=True)
    if graph:
        lib.qw_gpu_graph_free(graph)
    if group:
        lib.qw_gpu_group_free(group)
    gpu.close()
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, gpu, w, runner, host_layers, layers, out_local, group, out_full, world, barrier):
    """Same metric through the C-ABI calls a host program makes: every layer's
    q, k, v (this rank's heads) start in pinned HOST memory
    (h3_gpu_tensor_write_bf16), the ops run, and the layer's output -- the full
    gathered [rows, H*128] on every rank when the heads are sharded -- is read
    back to pinned host memory.  Host wall clock, max over ranks."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    lib = gpu.lib
    n = runner.n
    n_out = n * world if group else n
    nl = len(host_layers)
    pinned = []
    for sl in host_layers:
        bufs = []
        for x in sl:
            p = lib.qw_gpu_host_alloc(n * 2)
            if not p:
                return {"value": None, "unit": "TFLOP/s", "error": "pinned allocation failed"}
            C.memmove(p, x.ctypes.data, n * 2)
            bufs.append(p)
        pinned.append(bufs)
    out_host = lib.qw_gpu_host_alloc(n_out * 2)
    dq, dk, dv = gpu.new_bf16(n), gpu.new_bf16(n), gpu.new_bf16(n)

    def step():
        for i in range(w.layers):
            hq, hk, hv = pinned[i % nl]
            lib.h3_gpu_tensor_write_bf16(dq, hq, n)
            lib.h3_gpu_tensor_write_bf16(dk, hk, n)
            lib.h3_gpu_tensor_write_bf16(dv, hv, n)
            _, _, _, wqt, wkt = layers[i]
            if group:
                full = out_full[i & 1]
                runner.enqueue(dq, dk, dv, wqt, wkt, group=group, full=full)
                gpu.check(lib.qw_gpu_group_wait_output(group, full), "wait_output")
                gpu.check(lib.qw_gpu_tensor_read_async(gpu.handle, full, out_host, n_out), "read")
            else:
                runner.enqueue(dq, dk, dv, wqt, wkt, out=out_local)
                gpu.check(lib.qw_gpu_tensor_read_async(gpu.handle, out_local, out_host, n), "read")

    steps = max(1, min(args.steps, 5))
    gpu.begin(); step(); gpu.submit()
    barrier()
    before = gpu.stats().gpu_seconds
    t0 = time.perf_counter()
    gpu.begin()
    for _ in range(steps):
        step()
    gpu.submit()
    barrier()
    wall = time.perf_counter() - t0
    device_s = gpu.stats().gpu_seconds - before
    if world > 1:
        t = torch.tensor([wall, device_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        wall, device_s = float(t[0].item()), float(t[1].item())
    for bufs in pinned:
        for p in bufs:
            lib.qw_gpu_host_free(p)
    lib.qw_gpu_host_free(out_host)
    for t in (dq, dk, dv):
        gpu.free(t)
    flops = w.flops_per_layer() * w.layers * steps
    return {"value": flops / wall / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": 3 * n * 2 * w.layers * world,
            "d2h_bytes_per_step": n_out * 2 * w.layers * world,
            "ms_per_step": wall / steps * 1e3, "device_ms_per_step": device_s / steps * 1e3,
            "steps": steps,
            "note": f"host wall clock around {steps} steps incl. submit, max over ranks; byte "
                    f"counts summed over the {world} rank(s); {nl} distinct pinned layer input "
                    "sets cycled over the 32 layers"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", type=int, default=3, choices=[2, 3, 4, 5])
    ap.add_argument("--layers", type=int, default=0,
                    help="override the layer count (small captures under a profiler)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: attention epilogue stores to every rank (fused) or NCCL all-gather")
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
