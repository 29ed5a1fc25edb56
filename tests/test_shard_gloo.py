"""CPU, world_size 2 over gloo: the N > 1 host logic of the attention path.
Each rank runs the CPU oracle on its head slice of a small batched block-causal
workload, the slices are all-gathered rank-major (as NCCL lands them) and
interleaved; the result must equal the unsharded oracle bit for bit."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import oracle_lib as O
    from qwen_metal_b200 import sharding, workloads

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = workloads.Workload("gloo: text 24 + 6x6 image, batch 2", 2, 4, ((24, 0), (36, 1)),
                               ((6, 6),), text_len=(24, 9), text_pad=24, prologue=False)
        q, k, v, _, _ = workloads.layer_inputs(w, 0)
        tl = np.asarray(w.text_len, np.uint32)
        heads_local = w.heads // world
        ql, kl, vl = (sharding.shard_heads(x, rank, world) for x in (q, k, v))
        local, _ = O.sdpa(ql, kl, vl, w.limits(), w.batch, w.rows, w.rows, heads_local,
                          heads_local, workloads.SCALE, tl, w.text_pad)
        rows = w.batch * w.rows
        mine = torch.from_numpy(local.reshape(rows, heads_local * 128))
        landing = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(landing, mine)                       # rank-major, like ncclAllGather
        staged = np.stack([t.numpy() for t in landing])
        full = sharding.interleave(staged, rows, heads_local * 128, world)
        if rank == 0:
            ref, _ = O.sdpa(q, k, v, w.limits(), w.batch, w.rows, w.rows, w.heads, w.heads,
                            workloads.SCALE, tl, w.text_pad)
            ok = np.array_equal(full, ref.reshape(rows, w.heads * 128))
            open(os.path.join(result_dir, "ok"), "w").write("1" if ok else "0")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_head_sharding_over_gloo_world_2(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "ok").read() == "1"


def test_head_range_and_interleave():
    sys.path.insert(0, ROOT)
    from qwen_metal_b200 import sharding
    assert sharding.head_range(3, 8, 24) == (9, 12)
    with pytest.raises(ValueError):
        sharding.head_range(0, 5, 24)
    staged = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    full = sharding.interleave(staged, 3, 4, 2)
    assert full[1].tolist() == [4, 5, 6, 7, 16, 17, 18, 19]


def test_batch_group_layout():
    """rank = batch_index * head_groups + head_index; the batch items split first."""
    sys.path.insert(0, ROOT)
    from qwen_metal_b200 import sharding
    assert sharding.default_batch_groups(1, 2) == 1
    assert sharding.default_batch_groups(2, 2) == 2
    assert sharding.default_batch_groups(8, 2) == 2
    assert sharding.default_batch_groups(4, 1) == 1
    assert sharding.default_batch_groups(3, 2) == 1
    # 8 ranks, batch 2: ranks 0-3 take item 0, ranks 4-7 item 1, six heads each of 24
    seen = set()
    for rank in range(8):
        b, h, groups, b0, nb = sharding.layout(rank, 8, 2, 2)
        assert (groups, nb, b0) == (4, 1, b) and rank == b * 4 + h
        lo, hi = sharding.head_range(h, groups, 24)
        seen.update((b0, head) for head in range(lo, hi))
    assert seen == {(b, head) for b in range(2) for head in range(24)}   # every (item, head) once
    x = np.arange(2 * 3 * 24 * 128).reshape(2, 3, 24, 128)
    assert np.array_equal(sharding.shard(x, 6, 8, 2), x[1:2, :, 12:18])
    with pytest.raises(ValueError):
        sharding.layout(0, 8, 2, 3)


def _worker_batch_groups(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import oracle_lib as O
    from qwen_metal_b200 import sharding, workloads

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = workloads.Workload("gloo: text 24 + 6x6 image, batch 2", 2, 4, ((24, 0), (36, 1)),
                               ((6, 6),), text_len=(24, 9), text_pad=24, prologue=False)
        q, k, v, _, _ = workloads.layer_inputs(w, 0)
        groups = sharding.default_batch_groups(world, w.batch)
        _, head_index, head_groups, b0, nb = sharding.layout(rank, world, w.batch, groups)
        assert (groups, head_groups, nb) == (2, 1, 1)      # world 2: one item per rank, no exchange
        ql, kl, vl = (sharding.shard(x, rank, world, groups) for x in (q, k, v))
        tl = np.asarray(w.text_len[b0:b0 + nb], np.uint32)
        local, _ = O.sdpa(ql, kl, vl, w.limits(), nb, w.rows, w.rows, w.heads, w.heads,
                          workloads.SCALE, tl, w.text_pad)
        ref, _ = O.sdpa(q, k, v, w.limits(), w.batch, w.rows, w.rows, w.heads, w.heads,
                        workloads.SCALE, np.asarray(w.text_len, np.uint32), w.text_pad)
        ok = torch.tensor([int(np.array_equal(local, ref[b0:b0 + nb]))])
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if rank == 0:
            open(os.path.join(result_dir, "ok"), "w").write(str(int(ok.item())))
    finally:
        dist.destroy_process_group()


def test_batch_item_split_over_gloo_world_2(tmp_path):
    import torch.multiprocessing as mp
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_worker_batch_groups, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "ok").read() == "1"
