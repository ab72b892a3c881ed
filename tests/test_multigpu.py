"""The real NVLink path: one process per GPU, CUDA IPC peer tables, the flag protocol across devices, pull
reduce-scatter, fused kernel, push all-gather with its ticket tail and the dispatch to owning ranks at world 2, 4
and 8 (as many as the box has GPUs), each checked against the CPU oracle and then soaked for 500 replays whose
inputs change every replay (tests/multigpu_worker.py).  NVLS is off in NCCL for these runs and every wait in the
kernels is bounded.  Skipped on a single-GPU box."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_collectives_across_gpus(world):
    if _ngpu() < world:
        pytest.skip("needs %d GPUs" % world)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
           "--master-port", str(29610 + world), os.path.join(ROOT, "tests", "multigpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    sys.stdout.write(r.stdout[-4000:]); sys.stderr.write(r.stderr[-4000:])
    assert r.returncode == 0
    assert "MULTIGPU_OK" in r.stdout
