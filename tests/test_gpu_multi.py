"""GPU, needs >= 2 devices: head-sharded attention across one process per GPU
(NCCL gather and the push gather, heads over all ranks and batch items split
first), every rank's full gathered output against the CPU oracle.  Skipped on
a single-GPU box.  NVLS is switched off for NCCL so a rank that fails cannot take
multicast-bound memory of the others with it."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def device_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except (OSError, subprocess.TimeoutExpired):
        return 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_attention_world(tmp_path, world):
    if device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    worker = os.path.join(ROOT, "tests", "multi_rank_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), str(world), str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outputs.append(out)
    for r, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0 and os.path.exists(tmp_path / f"ok{r}"), f"rank {r}:\n{out[-3000:]}"


def test_push_wait_runs_out_when_a_rank_stays_away(tmp_path):
    """Failure detection of the head push, without a GPU fault: rank 1 does not join
    the second layer (host-side), rank 0's bounded flag wait expires, its submit
    reports it and its context keeps working.  NVLS off, plain peer stores."""
    if device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", QW_CUDA_GROUP_WAIT_MS="300")
    worker = os.path.join(ROOT, "tests", "multi_rank_timeout_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(tmp_path)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outputs.append(out)
    for r, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0 and os.path.exists(tmp_path / f"ok{r}"), f"rank {r}:\n{out[-3000:]}"
    assert "wait ran out" in open(tmp_path / "rank0_done").read()
