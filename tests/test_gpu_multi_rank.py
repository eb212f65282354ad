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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_serving_replay_finishes_every_request():
    """The multi-turn replay with the sessions dealt to two ranks (data-parallel attention, experts sharded):
    every request finishes, prefixes are reused, nothing is left unserved."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29671", "-m",
                          "ulacache_b200.experiments.online_serving", "--tiny", "--layers", "3", "--sessions", "6",
                          "--turns", "2,3", "--system-prefix", "256", "--median-input", "96", "--input-cap", "300",
                          "--output", "4,8", "--max-batch", "4", "--prefill-chunk", "64", "--device-records", "8192",
                          "--rate", "200"], cwd=repo, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["ranks"] == 2 and out["finished_requests"] == out["requests"] and out["rejected_requests"] == 0
    assert out["reused_prefix_tokens"] > 0 and out["unserved"] == 0
    assert out["ttft_s_p50"] > 0 and out["output_tokens_per_s"] > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_a_departed_rank_is_seen_on_the_host_before_the_next_launch():
    """A rank leaves between steps with nothing in flight; the other learns of it from the heartbeats before its
    next launch, launches nothing towards it, and its own GPU keeps working.  Plain peer stores, no multicast."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29691", "-m",
                          "ulacache_b200.benchmarks.rank_departure_check"], cwd=repo, env=env, capture_output=True,
                         text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    out = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert out["steps_before_departure_ok"] == 3 and out["detected"] == [1]
    assert out["launched_after_departure"] is False and out["local_gpu_ok_after"] and out["detect_s"] < 10
