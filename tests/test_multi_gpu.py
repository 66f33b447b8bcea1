"""Multi-process checks on real GPUs (skipped on a box with fewer than 2): launched as torchrun children."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(script, *args, nproc=2, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, script), *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["fused", "fused_allreduce", "nccl"])
def test_two_ranks_match_single_process_with_accumulation(mode):
    r = _torchrun("tests/multi_gpu/check_gpt_ranks_vs_single.py", "--mode", mode)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_full_model_free_running_ranks_match_single_process():
    """The benchmark's own step (124M parameters, 48 x 1024 tokens per rank, four sequences in rotation) with the host
    running ahead of the device: timing-dependent faults (a kernel of one stream overwriting what another still reads)
    only show at this size."""
    r = _torchrun("tests/multi_gpu/check_gpt_ranks_vs_single.py", "--mode", "fused", "--full", "--pool", "4", "--steps", "5", "--free-running")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_survivors_detect_a_rank_that_left_between_steps(tmp_path):
    """Host-made failure on real GPUs: the last rank raises between two steps (device idle) and leaves; the others
    learn of it from the heartbeat store before launching the next step's peer-waiting kernels, stop cleanly and name
    the failed rank; no device-side wait runs out. In-switch reduction is off for the run."""
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests/multi_gpu/check_failure_between_steps.py"), "--out", str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    outs = {k: (tmp_path / f"out{k}.txt").read_text() if (tmp_path / f"out{k}.txt").exists() else None for k in range(world)}
    assert r.returncode == 0, (outs, r.stdout[-1500:], r.stderr[-1500:])
    assert outs[world - 1].startswith("injected steps=3"), outs
    for k in range(world - 1):
        assert outs[k].startswith(f"detected:{world - 1} steps=3"), outs


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_optimizer_state_survives_save_and_resume(tmp_path):
    """Every rank saves its shard of the Muon momentum and the Adam moments; a fresh trainer that loads them continues
    on the trajectory of the run that never stopped."""
    r = _torchrun("tests/multi_gpu/check_checkpoint_resume.py", "--dir", str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
