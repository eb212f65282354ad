"""Two-rank check of the peer-memory protocols; needs two GPUs (skipped otherwise)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_peer_protocols():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29631", "-m",
                          "ulacache_b200.benchmarks.multi_rank_check"], cwd=repo, env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["all_ranks_ok"] and all(v for k, v in out.items() if not k.endswith("_error")), out
