"""One rank of the multi-GPU parity test (run as a child process, one per GPU):
sharded block-causal attention (prologue included, fixed-exponent softmax) with
(a) the NCCL all-gather + interleave over one batch group and (b) the push gather
of this library, once with the heads sharded over all ranks and once with the
batch items split first.  Every rank checks ITS gathered output, all head columns,
against the unsharded CPU oracle, so a wrong peer column is caught."""
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
                           ((96, 0), (400, 1)), ((20, 20),), text_len=(96, 31), text_pad=96)
    q, k, v, wq, wk = workloads.layer_inputs(w, 0)
    cos, sin = w.rope_tables()
    tl = np.asarray(w.text_len, np.uint32)
    rows_all = w.batch * w.rows
    qn = O.head_rms_norm(q, wq, rows_all, w.heads, workloads.EPS)
    kn = O.head_rms_norm(k, wk, rows_all, w.heads, workloads.EPS)
    for b in range(w.batch):
        qn[b], kn[b] = O.qk_rope(qn[b], kn[b], cos, sin, w.rows, w.heads)
    ref, _ = O.sdpa(qn, kn, v, w.limits(), w.batch, w.rows, w.rows, w.heads, w.heads,
                    workloads.SCALE, tl, w.text_pad)
    wqt, wkt = gpu.bf16(wq), gpu.bf16(wk)

    def check(bits, want, what):
        got = abi.bf16_to_f32(bits).astype(np.float64)
        diff = np.abs(got - want.ravel())
        rel = np.sqrt((diff ** 2).sum() / (want.astype(np.float64) ** 2).sum())
        assert diff.max() <= 2e-2 and diff.mean() <= 2e-3 and rel < 5e-3, (what, diff.max(), rel)

    for batch_groups in sorted({1, sharding.default_batch_groups(world, w.batch)}):
        gpu.check(lib.qw_gpu_group_set_batch_groups(group, batch_groups), "set_batch_groups")
        _, head_index, head_groups, b0, nb = sharding.layout(rank, world, w.batch, batch_groups)
        assert lib.qw_gpu_group_head_index(group) == head_index
        assert lib.qw_gpu_group_head_groups(group) == head_groups
        heads_local = w.heads // head_groups
        runner = workloads.LayerRunner(gpu, w, heads_local, batch_items=(b0, nb))
        qt, kt, vt = (gpu.bf16(sharding.shard(x, rank, world, batch_groups)) for x in (q, k, v))
        q_work, k_work = gpu.new_bf16(runner.n), gpu.new_bf16(runner.n)
        want = ref[b0:b0 + nb]                      # this batch group's items, ALL heads
        full_count = nb * w.rows * w.heads * 128
        full_a = None

        if batch_groups == 1:
            # (a) NCCL all-gather into a landing zone + interleave
            out_local = gpu.new_bf16(runner.n)
            full_a = gpu.new_bf16(full_count)
            gpu.begin()
            runner.enqueue(qt, kt, vt, wqt, wkt, out=out_local, q_work=q_work, k_work=k_work)
            gpu.check(lib.qw_gpu_group_all_gather_heads_bf16(group, full_a, out_local, nb * w.rows,
                                                             heads_local, 128), "all_gather")
            gpu.submit()
            check(gpu.read_bf16(full_a, full_count), want, "nccl gather")

        # (b) push gather: four layers alternating between two bound outputs, then
        # two layers replayed from a captured graph
        # (allocations of a few MB each: smaller ones may share a device memory block,
        # and a block can be opened through CUDA IPC only once per process)
        full_b = [gpu.new_bf16(max(full_count, 1 << 22)) for _ in range(2)]
        for t in full_b:
            gpu.check(lib.qw_gpu_group_bind_output(group, t), "bind")

        def layers(count):
            for i in range(count):
                runner.enqueue(qt, kt, vt, wqt, wkt, q_work=q_work, k_work=k_work, group=group,
                               full=full_b[i & 1])
        gpu.begin()
        layers(4)
        gpu.submit()
        for t in full_b:
            check(gpu.read_bf16(t, full_count), want, f"push gather, {batch_groups} batch group(s)")
        eager = gpu.read_bf16(full_b[1], full_count)
        assert np.array_equal(eager, gpu.read_bf16(full_b[0], full_count))
        if full_a is not None:
            assert np.array_equal(eager, gpu.read_bf16(full_a, full_count))
        gpu.begin()
        gpu.check(lib.qw_gpu_graph_begin(gpu.handle), "graph begin")
        layers(2)
        graph = lib.qw_gpu_graph_end(gpu.handle)
        assert graph, gpu.error()
        gpu.submit()
        zeros = np.zeros(full_count, np.uint16)
        for _ in range(3):
            # poison the buffers so that a replay that moved nothing would show
            for t in full_b:
                gpu.check(lib.h3_gpu_tensor_write_bf16(t, abi._ptr(zeros), full_count), "poison")
            gpu.begin()
            gpu.check(lib.qw_gpu_group_barrier(group), "barrier")   # every rank has poisoned
            gpu.check(lib.qw_gpu_graph_launch(gpu.handle, graph), "replay")
            gpu.submit()
            for t in full_b:
                assert np.array_equal(gpu.read_bf16(t, full_count), eager), "graph replay differs"
            gpu.begin()
            gpu.check(lib.qw_gpu_group_barrier(group), "barrier")   # every rank has read
            gpu.submit()
        lib.qw_gpu_graph_free(graph)

    # leave only after every rank is done with the peer mappings
    gpu.begin()
    gpu.check(lib.qw_gpu_group_barrier(group), "barrier")
    gpu.submit()
    lib.qw_gpu_group_free(group)
    gpu.close()
    open(os.path.join(workdir, f"ok{rank}"), "w").write("1")


if __name__ == "__main__":
    main()
