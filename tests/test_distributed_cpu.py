"""world_size-2 run of the data-parallel protocol on CPU (gloo); see multi_cpu_worker.py."""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_two_rank_protocol_on_gloo():
  env = dict(os.environ, OMP_NUM_THREADS="1")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", "29533", os.path.join(HERE, "multi_cpu_worker.py")]
  out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
  assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout
