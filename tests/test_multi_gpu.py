"""Multi-GPU checks of the shard + gather driver (csrc/dist.cu): N-column shards of a product reassembled by
te_b200_all_gather_columns, row blocks by te_b200_all_gather_rows, te_b200_gemm_f32_host_sharded, and attention sharded
by batch index.  One process per GPU through torch.distributed.run; skipped where fewer than two GPUs are visible (the
host-side shard logic is covered on CPU by tests/test_sharding_gloo.py)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4])
def test_column_and_batch_shards_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    env = dict(os.environ, NCCL_DEBUG="WARN")
    port = 29650 + world
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                        "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for rank in range(world):
        assert "rank %d ok" % rank in r.stdout
