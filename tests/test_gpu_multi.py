"""Multi-process, multi-GPU path (needs >= 2 GPUs on the box; skipped otherwise)."""

import os
import subprocess
import sys

import pytest

from helpers import free_port

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpu_count():
    import torch
    return torch.cuda.device_count()


def _torchrun(script, nproc, extra_env=None, timeout=600):
    # The workers size their own heaps: settings another test left in this process must not leak in.
    env = {k: v for k, v in os.environ.items()
           if not k.startswith("PCCL_") and k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(HERE, script)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_collectives_match_nccl(nproc):
    if _gpu_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    done = _torchrun("multi_gpu_worker.py", nproc)
    assert "MULTI_GPU_PASS" in done.stdout, done.stdout[-4000:] + done.stderr[-1500:]
