"""Row-sharded tables with one process per GPU (needs at least 2 GPUs; skipped otherwise)."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _gpus():
  import torch

  return torch.cuda.device_count()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_lookup_and_update_match_oracle(world):
  if _gpus() < world:
    pytest.skip(f"needs {world} GPUs")
  env = dict(os.environ, NCCL_NVLS_ENABLE="0")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), os.path.join(HERE, "multi_gpu_worker.py")]
  out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
  assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
  assert out.stdout.count("multi-gpu parity ok") == 3
