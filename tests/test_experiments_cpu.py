"""The experiment drivers' CPU parts: capacity model, scheduler study, serving trace builder."""
import json
import subprocess
import sys
import os

from ulacache_b200.experiments.capacity import organisations
from ulacache_b200.experiments.online_serving import build_trace
from ulacache_b200.experiments.scheduler_study import run, synthetic_trace

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_capacity_model_orders_the_organisations():
    org = organisations(device_gb=72, host_gb=128, ranks=8, layers=61, requests_per_rank=64)
    assert org["pooled"]["tp"] > 5 * org["hot_buffer"]["tp"] > 5 * org["replicated"]["tp"]
    assert org["pooled"]["dpa"] >= org["hot_buffer"]["dpa"] > org["replicated"]["dpa"]
    assert org["pooled"]["device_tokens_per_rank"] % 64 == 0 and org["pooled"]["host_tokens_per_rank"] % 64 == 0
    out = subprocess.run([sys.executable, "-m", "ulacache_b200.experiments.capacity"], cwd=REPO, capture_output=True,
                         text=True, timeout=120)
    rows = [json.loads(l) for l in out.stdout.splitlines()]
    assert len(rows) == 4 and {r["mode"] for r in rows} == {"tp8", "dpa8"}


def test_scheduler_study_runs_every_policy():
    steps = list(synthetic_trace(requests=3, steps=12, context=512, topk=64))
    rows = run(steps, capacity=256, per_request=96, record_bytes=656, layers=2)
    assert {r["policy"] for r in rows} == {"bucket_ring", "bitmap_ring", "exact_lru", "linked_list", "clock", "per_request"}
    ring, bitmap = (next(r for r in rows if r["policy"] == k) for k in ("bucket_ring", "bitmap_ring"))
    assert ring["hit_rate"] == bitmap["hit_rate"]           # the same decisions from two data structures
    lru = next(r for r in rows if r["policy"] == "exact_lru")
    assert 0.0 < lru["hit_rate"] < 1.0 and lru["overflow"] == 0 and lru["h2d_bytes_per_step"] > 0


def test_serving_trace_shape():
    tr = build_trace(sessions=5, turns_lo=2, turns_hi=3, system_prefix=128, median_input=64, sigma=0.8, input_cap=256,
                     out_lo=4, out_hi=8, rate=10.0, vocab=1000)
    assert 10 <= len(tr) <= 15 and all(a["arrival"] <= b["arrival"] for a, b in zip(tr, tr[1:]))
    first = [r for r in tr if r["session"] == 0]
    assert first[1]["prompt"][: len(first[0]["prompt"])] == first[0]["prompt"]            # turns extend their history
    assert all(r["prompt"][:128] == tr[0]["prompt"][:128] for r in tr)                     # shared system prefix


def test_frozen_workloads_are_reproducible_and_hash_pinned(tmp_path):
    import pytest
    from ulacache_b200.experiments import workloads as W

    a, b = str(tmp_path / "a.jsonl.gz"), str(tmp_path / "b.jsonl.gz")
    assert W.main(["prepare-conversations", a, "--sessions", "6", "--turns", "2,3", "--system-prefix", "128"]) == 0
    assert W.main(["prepare-conversations", b, "--sessions", "6", "--turns", "2,3", "--system-prefix", "128"]) == 0
    assert open(a, "rb").read() == open(b, "rb").read()                     # same seed, same bytes
    wl = W.load_workload(a)
    digest = wl["manifest"]["payload_sha256"]
    assert W.load_workload(b, digest)["manifest"]["records"] == len(wl["records"])
    with pytest.raises(ValueError):
        W.load_workload(a, "0" * 64)
    trace = W.as_trace(wl, vocab=1000)
    by_session = {}
    for r in trace:
        by_session.setdefault(r["session"], []).append(r)
    first = [v[0]["prompt"] for v in by_session.values()]
    assert all(p[:128] == first[0][:128] for p in first)                    # one shared system prefix
    for reqs in by_session.values():                                        # every turn extends the previous history
        for prev, nxt in zip(reqs, reqs[1:]):
            assert nxt["prompt"][: len(prev["prompt"])] == prev["prompt"] and len(nxt["prompt"]) > len(prev["prompt"]) + prev["max_new"]
    assert max(max(r["prompt"]) for r in trace) < 1000 and [r["arrival"] for r in trace] == sorted(r["arrival"] for r in trace)
    # a tampered payload is refused
    import gzip
    raw = gzip.decompress(open(a, "rb").read()).replace(b'"max_new":', b'"max_new": ', 1)
    open(a, "wb").write(gzip.compress(raw, mtime=0))
    with pytest.raises(ValueError):
        W.load_workload(a)
    docs = str(tmp_path / "docs.jsonl.gz")
    assert W.main(["prepare-documents", docs, "--count", "200", "--mean-tokens", "98000"]) == 0
    s = W.summary(W.load_workload(docs))
    assert s["records"] == 200 and 80000 < s["prompt_tokens_mean"] < 120000 and s["prompt_tokens_max"] <= 262144
    assert len(W.expand_prompt(W.load_workload(docs)["records"][0])) == W.load_workload(docs)["records"][0]["prompt_tokens"]


def test_results_csv_grows_rows_and_columns(tmp_path):
    import csv
    from ulacache_b200.utils import append_result_csv

    path = str(tmp_path / "results.csv")
    append_result_csv(path, {"experiment": "decode_sweep", "global_batch": 64, "tokens_per_s": 2467.0})
    append_result_csv(path, {"experiment": "decode_sweep", "global_batch": 128, "tokens_per_s": 4495.0})
    append_result_csv(path, {"experiment": "decode_sweep", "global_batch": 256, "tokens_per_s": 7627.0, "clocks": {"sm_mhz": 1965}})
    rows = list(csv.DictReader(open(path, newline="")))
    assert [r["global_batch"] for r in rows] == ["64", "128", "256"] and rows[0]["clocks"] == "" and "1965" in rows[2]["clocks"]


def test_captured_traces_are_validated_and_composed(tmp_path):
    import numpy as np
    import pytest
    from ulacache_b200.experiments import scheduler_study as S

    def capture(path, steps, layers, seed):
        rng = np.random.default_rng(seed)
        rows = [(s, l, int(i)) for s in range(steps) for l in range(layers) for i in rng.integers(1, 1000, 8)]
        np.save(path, np.array(rows, dtype=np.int32))
        return path

    a = capture(str(tmp_path / "rank0.npy"), 5, 2, 0)
    b = capture(str(tmp_path / "rank1.npy"), 4, 2, 1)
    rec = S.validate_capture(a, layers=2)
    assert rec["steps"] == 5 and rec["layers"] == 2 and rec["triples"] == 80 and rec["ids_per_step_layer_min"] == 8
    S.validate_capture(a, expected_sha256=rec["sha256"])
    with pytest.raises(ValueError):
        S.validate_capture(a, expected_sha256="0" * 64)
    with pytest.raises(ValueError):
        S.validate_capture(a, layers=3)
    holes = np.load(a)
    np.save(str(tmp_path / "holes.npy"), holes[~((holes[:, 0] == 2) & (holes[:, 1] == 1))])
    with pytest.raises(ValueError):
        S.validate_capture(str(tmp_path / "holes.npy"))
    out = S.compose_rank_traces([a, b], str(tmp_path / "both.npy"), id_space_per_rank=1000)
    both = np.load(out["path"])
    assert out["steps"] == 4 and out["ranks"] == 2 and both.shape[0] == 4 * 2 * 8 * 2
    assert int(both[:, 2].max()) >= 1000 and out["sources"][1]["id_offset"] == 1000
    step0 = both[(both[:, 0] == 0) & (both[:, 1] == 0)][:, 2]
    assert (step0 < 1000).sum() == 8 and (step0 >= 1000).sum() == 8           # both ranks' requests in one step
    with pytest.raises(ValueError):
        S.compose_rank_traces([a, b], str(tmp_path / "bad.npy"), id_space_per_rank=500)
    # the composed load replays through the policy oracle like any other trace
    rows = S.run(list(S.trace_from_file(out["path"])), 64, per_request=8, record_bytes=656, layers=1)
    assert rows and all(r["steps"] == 4 for r in rows)
