"""One rank of the multi-GPU parity test (run as a child process, one per GPU):
head-sharded block-causal attention with (a) the NCCL all-gather + interleave and
(b) the fused peer-store gather, both against the unsharded CPU oracle."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    rank, world, workdir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    import ctypes as C
    import oracle_lib as O
    from qwen_metal_b200 import abi, sharding, workloads

    gpu = abi.Gpu(rank)
    lib = gpu.lib
    id_path = os.path.join(workdir, "nccl_id")
    ident = np.zeros(128, np.uint8)
    err = C.create_string_buffer(256)
    if rank == 0:
        assert lib.qw_gpu_group_new_id(abi._ptr(ident), err, 256), err.value
        with open(id_path + ".tmp", "wb") as f:
            f.write(ident.tobytes())
        os.rename(id_path + ".tmp", id_path)
    else:
        deadline = time.time() + 60
        while not os.path.exists(id_path):
            assert time.time() < deadline, "rank 0 never published the group id"
            time.sleep(0.05)
        ident = np.frombuffer(open(id_path, "rb").read(), np.uint8).copy()
    group = lib.qw_gpu_group_join(gpu.handle, abi._ptr(ident), rank, world, err, 256)
    assert group, err.value

    w = workloads.Workload("multi: text 96 + 20x20 image, batch 2 with key padding", 2, 4 * world,
                           ((96, 0), (400, 1)), ((20, 20),), text_len=(96, 31), text_pad=96,
                           prologue=False)
    q, k, v, _, _ = workloads.layer_inputs(w, 0)
    heads_local = w.heads // world
    runner = workloads.LayerRunner(gpu, w, heads_local)
    qt, kt, vt = (gpu.bf16(sharding.shard_heads(x, rank, world)) for x in (q, k, v))
    rows = w.batch * w.rows
    full_count = rows * w.heads * 128
    tl = np.asarray(w.text_len, np.uint32)
    ref, _ = O.sdpa(q, k, v, w.limits(), w.batch, w.rows, w.rows, w.heads, w.heads,
                    workloads.SCALE, tl, w.text_pad)

    def check(bits, what):
        got = abi.bf16_to_f32(bits).astype(np.float64)
        diff = np.abs(got - ref.ravel())
        rel = np.sqrt((diff ** 2).sum() / (ref.astype(np.float64) ** 2).sum())
        assert diff.max() <= 2e-2 and diff.mean() <= 2e-3 and rel < 5e-3, (what, diff.max(), rel)

    # (a) NCCL all-gather into a landing zone + interleave
    out_local = gpu.new_bf16(runner.n)
    full_a = gpu.new_bf16(full_count)
    gpu.begin()
    runner.enqueue(qt, kt, vt, out=out_local)
    gpu.check(lib.qw_gpu_group_all_gather_heads_bf16(group, full_a, out_local, rows, heads_local,
                                                     128), "all_gather")
    gpu.submit()
    check(gpu.read_bf16(full_a, full_count), "nccl gather")

    # (b) fused: the attention epilogue stores into every rank's bound output, twice
    full_b = [gpu.new_bf16(full_count) for _ in range(2)]
    for t in full_b:
        gpu.check(lib.qw_gpu_group_bind_output(group, t), "bind")
    gpu.begin()
    for t in full_b:
        runner.enqueue(qt, kt, vt, group=group, full=t)
    gpu.submit()
    for t in full_b:
        check(gpu.read_bf16(t, full_count), "fused gather")
    assert np.array_equal(gpu.read_bf16(full_b[0], full_count), gpu.read_bf16(full_a, full_count))

    # leave only after every rank is done with the peer mappings
    gpu.begin()
    gpu.check(lib.qw_gpu_group_barrier(group), "barrier")
    gpu.submit()
    lib.qw_gpu_group_free(group)
    gpu.close()
    open(os.path.join(workdir, f"ok{rank}"), "w").write("1")


if __name__ == "__main__":
    main()
