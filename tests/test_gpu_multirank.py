"""GPU, needs >= 2 devices: the EP > 1 path (CUDA-IPC arenas, count exchange, pull dispatch, push
return, generation flags) through tests/ep_worker.py under torch.distributed.run."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_parity(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + world), str(ROOT / "tests" / "ep_worker.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    for scenario in ("mixed planners", "overflow reporting passed", "headline shape", "absent rank"):
        assert scenario in done.stdout, scenario
