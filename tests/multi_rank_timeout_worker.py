"""One rank of the push-timeout test (run as a child process, one per GPU, world 2).

Rank 1 runs the first sharded layer and then stays away from the second one (it
keeps its process and its GPU context alive, with nothing in flight).  Rank 0 runs
both: the push behind its second layer waits for rank 1's "your stores may start"
flag, which never comes; after the short budget set through
QW_CUDA_GROUP_WAIT_MS the kernel records the expiry, skips the stores to that peer
and returns, and h3_gpu_submit reports it.  Nothing faults, traps or hangs; the
failure is a rank that does not join, made on the host."""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def wait_for(path, seconds=120):
    deadline = time.time() + seconds
    while not os.path.exists(path):
        assert time.time() < deadline, f"{path} never appeared"
        time.sleep(0.05)


def main():
    rank, world, workdir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    assert world == 2
    import ctypes as C
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
        wait_for(id_path)
        ident = np.frombuffer(open(id_path, "rb").read(), np.uint8).copy()
    group = lib.qw_gpu_group_join(gpu.handle, abi._ptr(ident), rank, world, err, 256)
    assert group, err.value

    w = workloads.Workload("timeout: text 32 + 16x16 image", 1, 8, ((32, 0), (256, 1)), ((16, 16),),
                           prologue=False)
    q, k, v, _, _ = workloads.layer_inputs(w, 0)
    runner = workloads.LayerRunner(gpu, w, w.heads // 2)
    qt, kt, vt = (gpu.bf16(sharding.shard(x, rank, world, 1)) for x in (q, k, v))
    full = [gpu.new_bf16(1 << 22) for _ in range(2)]
    for t in full:
        gpu.check(lib.qw_gpu_group_bind_output(group, t), "bind")

    # layer 1: both ranks take part, everything completes
    gpu.begin()
    runner.enqueue(qt, kt, vt, group=group, full=full[0])
    gpu.submit()
    open(os.path.join(workdir, f"layer1_{rank}"), "w").write("1")
    wait_for(os.path.join(workdir, f"layer1_{1 - rank}"))

    if rank == 0:
        # layer 2 on the other bound output: rank 1 never starts it
        t0 = time.time()
        gpu.begin()
        runner.enqueue(qt, kt, vt, group=group, full=full[1])
        ok = lib.h3_gpu_submit(gpu.handle)
        waited = time.time() - t0
        message = gpu.error()
        assert ok == 0 and "wait ran out" in message, (ok, message)
        assert waited < 30, waited
        # the context is still usable: an ordinary launch works
        gpu.begin()
        runner.enqueue(qt, kt, vt)
        gpu.submit()
        open(os.path.join(workdir, "rank0_done"), "w").write(message)
    else:
        wait_for(os.path.join(workdir, "rank0_done"))   # alive, idle, nothing in flight
    lib.qw_gpu_group_free(group)
    gpu.close()
    open(os.path.join(workdir, f"ok{rank}"), "w").write("1")


if __name__ == "__main__":
    main()
