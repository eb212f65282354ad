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


def trace_from_frames(path: str, layer: int = 0):
    """Replay input out of a framed capture (``capture_decode_frames``): per step the lookups of one layer as
    (ids, requests), current records and padding removed, request identity kept."""
    import numpy as np
    import torch
    from ..telemetry.sparse_trace import frames_to_lookups

    z = np.load(path)
    chunk = dict(frame_count=int(z["selected"].shape[0]), selected=torch.from_numpy(z["selected"]),
                 current=torch.from_numpy(z["current"]), seen=torch.from_numpy(z["seen"]))
    yield from frames_to_lookups(chunk, z["query_requests"].tolist(), group=layer)


def capture_decode_frames(path: str, *, steps: int, batch: int, prompt_len: int, layers: int, tiny: bool):
    """Like ``capture_decode_trace`` but framed: every step stores, per layer, each row's selection AND the record
    the row is writing, plus the allocation events, in one ``.npz`` (selected [steps, layers, batch, topk],
    current [steps, layers, batch], seen, epochs, events, query_requests).  Returns the receipt."""
    import numpy as np
    import torch
    from ..models.dsa_moe import DsaMoeConfig
    from ..serving.engine import DecodeEngine
    from ..telemetry.sparse_trace import FramedSparseTrace, SparseTraceGeometry

    cfg = DsaMoeConfig().tiny(layers=layers, topk=128) if tiny else DsaMoeConfig(layers=layers, unique_layer_weights=min(layers, 4))
    eng = DecodeEngine(cfg, batch=batch, prompt_len=prompt_len, max_new_tokens=steps + 8, mode="dpa", use_graph=False)
    eng.fill_synthetic()
    geo = SparseTraceGeometry(groups=cfg.layers, query_rows=batch, topk=cfg.topk, frames=steps, chunk_frames=steps,
                              event_capacity=max(64, 2 * steps * batch))
    rec = FramedSparseTrace(geo, device=eng.device)
    rec.start()
    for step in range(steps):
        eng.model.record_selections, eng.model.record_current = [], []
        rec.begin_frame(batch)
        eng.step_device()
        for lay, (sel, cur) in enumerate(zip(eng.model.record_selections, eng.model.record_current)):
            rec.observe(lay, sel, cur.reshape(-1)[:batch], step)
        rec.observe_event(eng.model.record_current[0], release=False)
    eng.model.record_selections = eng.model.record_current = None
    eng.check()
    chunk = rec.drain_chunk()
    events = rec.event_snapshot()
    rec.stop()
    eng.close()
    np.savez(path, selected=chunk["selected"].numpy(), current=chunk["current"].numpy(), seen=chunk["seen"].numpy(),
             epochs=chunk["epochs"].numpy(), events=events.numpy(), query_requests=np.arange(batch, dtype=np.int64))
    saved = path if path.endswith(".npz") else path + ".npz"
    return dict(path=saved, sha256=_sha256(saved), steps=steps, layers=cfg.layers, batch=batch, events=int(events.shape[0]))


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


def _sha256(path: str) -> str:
    import hashlib

    with open(path, "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def validate_capture(path: str, *, expected_sha256: str = None, layers: int = None) -> dict:
    """Checks of a captured trace (int32 triples step, layer, id) before any policy is replayed over it: the file
    hashes to what the capture recorded, steps run from 0 without gaps, every step has every layer, ids are
    positive.  Returns the receipt that goes beside the results.

    Reference: scripts/7_5_scheduler/_runtime/validate_capture.py:19 (hash-pinned chunks, shape and positivity
    checks, coverage of every forward)."""
    import numpy as np

    digest = _sha256(path)
    if expected_sha256 is not None and digest != expected_sha256:
        raise ValueError("the captured trace changed since it was recorded")
    data = np.load(path)
    if data.ndim != 2 or data.shape[1] != 3 or data.dtype != np.int32 or data.shape[0] == 0:
        raise ValueError("a captured trace is a non-empty int32 array of (step, layer, id) triples")
    steps, lays, ids = data[:, 0], data[:, 1], data[:, 2]
    if int(ids.min()) <= 0:
        raise ValueError("captured ids must be positive (padding does not belong in a trace)")
    n_steps = int(steps.max()) + 1
    seen_layers = sorted(set(int(x) for x in np.unique(lays)))
    if layers is not None and seen_layers != list(range(layers)):
        raise ValueError(f"the trace covers layers {seen_layers}, not 0..{layers - 1}")
    pairs = set(zip(steps.tolist(), lays.tolist()))
    missing = [(s_, l_) for s_ in range(n_steps) for l_ in seen_layers if (s_, l_) not in pairs]
    if missing:
        raise ValueError(f"the trace misses (step, layer) {missing[:4]} ...: not every forward was captured")
    per = np.bincount(steps.astype(np.int64) * len(seen_layers) + np.searchsorted(seen_layers, lays))
    return dict(path=path, sha256=digest, steps=n_steps, layers=len(seen_layers), triples=int(data.shape[0]),
                ids_per_step_layer_min=int(per.min()), ids_per_step_layer_max=int(per.max()), id_max=int(ids.max()))


def compose_rank_traces(paths, out_path: str, *, id_space_per_rank: int) -> dict:
    """One larger shared-pool load out of independent per-rank captures: rank r's ids get the fixed offset
    ``r * id_space_per_rank`` (identity inside a rank is preserved), steps are aligned at 0 and cut to the shortest
    capture.  A construction from traces, not a capture of a bigger batch; the receipt names every source by hash.

    Reference: scripts/7_5_scheduler/_runtime/trace_data.py:18 (rank-offset UIDs, hashed sources)."""
    import numpy as np

    parts, sources, n_steps = [], [], None
    for rank, path in enumerate(paths):
        rec = validate_capture(path)
        data = np.load(path).astype(np.int64)
        if int(data[:, 2].max()) >= id_space_per_rank:
            raise ValueError(f"{path}: ids exceed the per-rank id space")
        data[:, 2] += rank * id_space_per_rank
        if data[:, 2].max() >= 2 ** 31:
            raise ValueError("composed ids no longer fit int32")
        n_steps = rec["steps"] if n_steps is None else min(n_steps, rec["steps"])
        parts.append(data)
        sources.append(dict(rank=rank, path=path, sha256=rec["sha256"], id_offset=rank * id_space_per_rank, steps=rec["steps"]))
    both = np.concatenate([p[p[:, 0] < n_steps] for p in parts]).astype(np.int32)
    order = np.lexsort((both[:, 1], both[:, 0]))
    np.save(out_path, both[order])
    final = out_path if out_path.endswith(".npy") else out_path + ".npy"
    return dict(path=final, sha256=_sha256(final), steps=n_steps, ranks=len(parts), sources=sources,
                construction="trace-driven composition of per-rank captures (not a capture at the larger batch)")


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


def _load(path: str):
    """A saved trace by its form: ``.npz`` = framed capture, ``.npy`` = (step, layer, id) triples."""
    return trace_from_frames(path) if path.endswith(".npz") else trace_from_file(path)


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
    ap.add_argument("--framed", action="store_true",
                    help="with --capture: framed capture (.npz: selections, current records, events, request of every row)")
    ap.add_argument("--full-width", action="store_true", help="capture from the full-width model instead of the tiny one")
    ap.add_argument("--gpu-timing", action="store_true", help="also replay through the device policies with per-step timing")
    ap.add_argument("--validate", default="", help="check a captured trace and print its receipt")
    ap.add_argument("--compose", default="", help="comma-separated per-rank traces to compose into one load")
    ap.add_argument("--compose-to", default="composed_trace.npy")
    ap.add_argument("--id-space-per-rank", type=int, default=1 << 24)
    args = ap.parse_args()
    if args.validate:
        print(json.dumps({"experiment": "scheduler_study_validate", **validate_capture(args.validate)}))
        return
    if args.compose:
        rec = compose_rank_traces(args.compose.split(","), args.compose_to, id_space_per_rank=args.id_space_per_rank)
        print(json.dumps({"experiment": "scheduler_study_compose", **rec}))
        args.trace = rec["path"]
    if args.capture and args.framed:
        rec = capture_decode_frames(args.capture_to, steps=args.capture, batch=args.capture_batch,
                                    prompt_len=args.capture_prompt, layers=args.capture_layers, tiny=not args.full_width)
        print(json.dumps({"experiment": "scheduler_study_frames", **rec}))
        args.trace = rec["path"]
    elif args.capture:
        n = capture_decode_trace(args.capture_to, steps=args.capture, batch=args.capture_batch, prompt_len=args.capture_prompt,
                                 layers=args.capture_layers, tiny=not args.full_width)
        print(json.dumps({"experiment": "scheduler_study", "captured_triples": n, "trace": args.capture_to,
                          "steps": args.capture, "layers": args.capture_layers}))
        args.trace = args.capture_to
    for cap in (int(c) for c in args.capacity.split(",")):
        if args.gpu_timing:
            steps = [ids for ids, _ in (_load(args.trace) if args.trace else
                                        synthetic_trace(requests=args.requests, steps=args.steps, context=args.context, topk=args.topk))]
            id_space = max(max(s) for s in steps if s) + 1
            for row in gpu_policy_timing(steps, cap, id_space):
                print(json.dumps({"experiment": "scheduler_study_gpu", **row}))
        if args.trace:
            steps = list(_load(args.trace))
        else:
            steps = list(synthetic_trace(requests=args.requests, steps=args.steps, context=args.context, topk=args.topk))
        for row in run(steps, cap, per_request=max(1, cap // max(1, args.requests)), record_bytes=656, layers=args.layers):
            print(json.dumps({"experiment": "scheduler_study", **row}))


if __name__ == "__main__":
    main()
