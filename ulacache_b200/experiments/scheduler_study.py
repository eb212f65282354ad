"""Replacement-policy study: replay a selection trace (recorded with
``telemetry.GpuSparseTraceRecorder`` or synthesised) through every policy and report hit rates and
host->device traffic at several device-tier sizes.

    python -m ulacache_b200.experiments.scheduler_study --trace trace.npy --capacity 65536,262144
    python -m ulacache_b200.experiments.scheduler_study --synthetic --requests 16 --steps 200
    python -m ulacache_b200.experiments.scheduler_study --capture 24 --capture-to trace.npy --gpu-timing

``--capture N`` records the selections of N decode steps of a running engine (every layer, through the
device trace ring of ``telemetry.GpuSparseTraceRecorder``) and replays them; ``--gpu-timing`` also replays
the trace through the device policies (exact LRU, linked list, sequential and parallel presence-bitmap
rings) and reports the device time per step of each beside its hit rate.

The synthetic trace models sparse attention selections: per request a slowly drifting hot set
(attention sinks + recent window + a few persistent heavy hitters) plus a uniformly random tail.

Reference: scripts/7_5_scheduler/run.py, _runtime/replay.py:1-559, reference.py + reference.cpp
(CPU oracle), README.md:25-36 (21 Index groups, page 64, 1,048,576-record pool).
"""
from __future__ import annotations

import argparse
import json
import random

from ..eviction.oracle import POLICY_KINDS, PolicyOracle


def synthetic_trace(*, requests: int, steps: int, context: int, topk: int, seed: int = 0, hot_fraction: float = 0.7,
                    drift: float = 0.02):
    """Yields per step (ids, request of each id); record id = request * context + position."""
    rng = random.Random(seed)
    n_hot = int(topk * hot_fraction)
    hot = [rng.sample(range(context), n_hot) for _ in range(requests)]
    for _ in range(steps):
        ids, reqs = [], []
        for r in range(requests):
            for j in range(n_hot):
                if rng.random() < drift:
                    hot[r][j] = rng.randrange(context)
            sel = set(hot[r])
            while len(sel) < topk:
                sel.add(rng.randrange(context))
            ids.extend(r * context + p for p in sorted(sel))
            reqs.extend([r] * len(sel))
        yield ids, reqs


def trace_from_file(path: str, layer: int = 0):
    from ..telemetry.sparse_trace import load_trace

    tr = load_trace(path)
    for (step, lay) in sorted(tr):
        if lay == layer:
            ids = sorted(set(int(x) for x in tr[(step, lay)] if x > 0))
            yield ids, [0] * len(ids)


def capture_decode_trace(path: str, *, steps: int, batch: int, prompt_len: int, layers: int, tiny: bool, layer: int = 0):
    """Run ``steps`` eager decode steps of an engine filled with synthetic history, append every layer's
    selection to the device trace ring, drain it between steps and save the trace.  Returns the triples saved."""
    import torch
    from ..models.dsa_moe import DsaMoeConfig
    from ..serving.engine import DecodeEngine
    from ..telemetry.sparse_trace import GpuSparseTraceRecorder

    cfg = DsaMoeConfig().tiny(layers=layers, topk=128) if tiny else DsaMoeConfig(layers=layers, unique_layer_weights=min(layers, 4))
    eng = DecodeEngine(cfg, batch=batch, prompt_len=prompt_len, max_new_tokens=steps + 8, mode="dpa", use_graph=False)
    eng.fill_synthetic()
    rec = GpuSparseTraceRecorder(eng.device, capacity_triples=batch * cfg.topk * cfg.layers * 2)
    for step in range(steps):
        eng.model.record_selections = []
        eng.step_device()
        for lay, sel in enumerate(eng.model.record_selections):
            rec.record(step, lay, sel)
        rec.drain()
    eng.model.record_selections = None
    eng.check()
    n = rec.save(path)
    eng.close()
    if rec.dropped:
        raise RuntimeError(f"the trace ring dropped {rec.dropped} triples")
    return n


def gpu_policy_timing(steps, capacity: int, id_space: int):
    """Replay ``steps`` (lists of distinct ids) through the device policies; CUDA events around each step."""
    import torch
    from ..eviction import ExactLruPolicy, LinkedListLruPolicy, ParallelPresenceRingPolicy, PresenceRingPolicy

    rows = []
    for name, cls in (("exact_lru", ExactLruPolicy), ("linked_list", LinkedListLruPolicy),
                      ("presence_ring_one_thread", PresenceRingPolicy), ("presence_ring_parallel", ParallelPresenceRingPolicy)):
        pol = cls(capacity, id_space, "cuda")
        times = []
        for ids in steps:
            t = torch.tensor(ids, dtype=torch.int32, device="cuda")
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            pol.step(t)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        times.sort()
        tot = pol.totals
        rows.append({"policy": name, "capacity_records": capacity, "steps": len(steps),
                     "hit_rate": round(tot["hits"] / max(1, tot["hits"] + tot["misses"]), 4), "evictions": tot["evictions"],
                     "median_us_per_step": round(times[len(times) // 2], 1), "p90_us_per_step": round(times[int(len(times) * 0.9)], 1),
                     "timing": "CUDA events around the policy's launches of one step (host-side orchestration included)"})
    return rows


def run(steps_iter, capacity: int, per_request: int, record_bytes: int, layers: int):
    sims = {k: PolicyOracle(k, capacity, per_request=per_request) for k in POLICY_KINDS}
    n_steps = 0
    for ids, reqs in steps_iter:
        n_steps += 1
        for kind, sim in sims.items():
            sim.step(ids, reqs if kind == "per_request" else None)
    rows = []
    for kind, sim in sims.items():
        t = sim.totals
        rows.append({"policy": kind, "capacity_records": capacity, "steps": n_steps, "hit_rate": round(sim.hit_rate(), 4),
                     "misses": t["misses"], "evictions": t["evictions"], "overflow": t["overflow"],
                     "h2d_bytes_per_step": t["misses"] * record_bytes * layers // max(1, n_steps)})
        sim.close()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--trace", default="")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--requests", type=int, default=8)
    ap.add_argument("--steps", type=int, default=60)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--topk", type=int, default=512)
    ap.add_argument("--capacity", default="4096,8192,16384")
    ap.add_argument("--layers", type=int, default=1, help="layers of one residency group (bytes moved per miss)")
    ap.add_argument("--capture", type=int, default=0, help="record this many decode steps of a running engine first")
    ap.add_argument("--capture-to", default="captured_trace.npy")
    ap.add_argument("--capture-batch", type=int, default=4)
    ap.add_argument("--capture-prompt", type=int, default=4096)
    ap.add_argument("--capture-layers", type=int, default=4)
    ap.add_argument("--full-width", action="store_true", help="capture from the full-width model instead of the tiny one")
    ap.add_argument("--gpu-timing", action="store_true", help="also replay through the device policies with per-step timing")
    args = ap.parse_args()
    if args.capture:
        n = capture_decode_trace(args.capture_to, steps=args.capture, batch=args.capture_batch, prompt_len=args.capture_prompt,
                                 layers=args.capture_layers, tiny=not args.full_width)
        print(json.dumps({"experiment": "scheduler_study", "captured_triples": n, "trace": args.capture_to,
                          "steps": args.capture, "layers": args.capture_layers}))
        args.trace = args.capture_to
    for cap in (int(c) for c in args.capacity.split(",")):
        if args.gpu_timing:
            steps = [ids for ids, _ in (trace_from_file(args.trace) if args.trace else
                                        synthetic_trace(requests=args.requests, steps=args.steps, context=args.context, topk=args.topk))]
            id_space = max(max(s) for s in steps if s) + 1
            for row in gpu_policy_timing(steps, cap, id_space):
                print(json.dumps({"experiment": "scheduler_study_gpu", **row}))
        if args.trace:
            steps = list(trace_from_file(args.trace))
        else:
            steps = list(synthetic_trace(requests=args.requests, steps=args.steps, context=args.context, topk=args.topk))
        for row in run(steps, cap, per_request=max(1, cap // max(1, args.requests)), record_bytes=656, layers=args.layers):
            print(json.dumps({"experiment": "scheduler_study", **row}))


if __name__ == "__main__":
    main()
