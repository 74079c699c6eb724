"""Multi-GPU check of the square-block partition of the dense operator (DenseGridShard) with the real kernels
and NCCL: needs four GPUs in one box, so it is skipped elsewhere; the partition logic itself is covered on the
CPU by test_shard_gloo.py."""
import os
import subprocess
import sys

import pytest


@pytest.mark.gpu
def test_square_block_shards_on_four_gpus():
    import torch
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    port = 36000 + os.getpid() % 2000
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(here, "grid_shard_check.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "grid-ok" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
