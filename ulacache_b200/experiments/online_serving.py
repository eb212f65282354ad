"""Multi-turn tiered serving replay on one GPU: sessions of several turns share a system prefix,
every turn appends a log-normally distributed new input to the session's history, arrivals are
Poisson.  The KV pool is sized to a multiple of the device tier so that it spills to host memory;
the radix tree reuses the shared prefix and each session's earlier turns.

    python -m ulacache_b200.experiments.online_serving --sessions 16 --layers 4 --system-prefix 1024

Prints one JSON line: admitted requests, KV capacity, TTFT / TPOT p50 / p99, output tokens/s,
prefix reuse, promotions and evictions.  (Scaled down by flags: the full study is 512 sessions of
4-12 turns, a 4K-token shared prefix, median-2K inputs capped at 16K, 256-1024 output tokens, total
KV three times the aggregate HBM.)

Reference: scripts/7_1_online/run.py:37-736 (multi-turn replay over SSE, TTFT/TPOT percentiles).
"""
from __future__ import annotations

import argparse
import json
import math
import random


def ttft(args):
    """Time to first token of one request: the prompt goes through the model in chunks of
    ``--prefill-chunk`` rows (every row selects and attends with its own causal length), then one token
    is sampled.  Wall clock around the chunks with a synchronize on both sides, after a warm-up request of
    two chunks; reported with the chunk count and the per-chunk time."""
    import time

    import torch
    from ..models.dsa_moe import DsaMoeConfig
    from ..serving.server import ServingEngine

    n = args.ttft_prompt
    cfg = (DsaMoeConfig().tiny(layers=args.layers, topk=256) if args.tiny
           else DsaMoeConfig(layers=args.layers, unique_layer_weights=min(args.layers, args.unique_layers)))
    records = (n + 4 * args.prefill_chunk + 4096) // 64 * 64
    srv = ServingEngine(cfg, max_batch=args.max_batch, max_context=n + 64, device_records=records, host_records=0,
                        prefill_chunk=args.prefill_chunk)
    import random

    rng = random.Random(0)
    warm = [rng.randrange(cfg.vocab) for _ in range(min(n, 2 * args.prefill_chunk))]
    srv.submit(0, warm, 1, 0.0)
    while srv.busy():
        srv.step()
    torch.cuda.synchronize()
    prompt = [rng.randrange(cfg.vocab) for _ in range(n)]
    t0 = time.perf_counter()
    srv.clock = lambda: time.perf_counter() - t0
    srv.finished.clear()
    srv.submit(1, prompt, 1, 0.0)
    steps = 0
    sections = None
    while srv.busy():
        if args.sections and steps == args.sections:        # per-section device time of ONE chunk
            srv.model.enable_profile(True)
        srv.step()
        if args.sections and steps == args.sections:
            sections = {k: round(v, 2) for k, v in srv.model.profile_summary().items()}
            srv.model.enable_profile(False)
        steps += 1
    torch.cuda.synchronize()
    r = srv.finished[-1]
    if sections is not None:
        print(json.dumps(dict(experiment="ttft_chunk_sections_ms", chunk_index=args.sections, sections=sections)))
    out = dict(experiment="ttft", prompt_tokens=n, prefill_chunk=args.prefill_chunk, layers=cfg.layers,
               distinct_layer_weight_sets_resident=cfg.unique_layer_weights or cfg.layers, chunks=steps,
               ttft_s=round(r.first_token_time - r.arrival, 4),
               ms_per_chunk=round(1e3 * (r.first_token_time - r.arrival) / max(1, steps), 2),
               prompt_tokens_per_s=round(n / (r.first_token_time - r.arrival), 1), model="tiny" if args.tiny else "full width")
    print(json.dumps(out))
    srv.close()


def build_trace(*, sessions, turns_lo, turns_hi, system_prefix, median_input, sigma, input_cap, out_lo, out_hi, rate,
                vocab, seed=0):
    rng = random.Random(seed)
    system = [rng.randrange(vocab) for _ in range(system_prefix)]
    t, reqs, rid = 0.0, [], 0
    histories = [list(system) for _ in range(sessions)]
    turns = [rng.randint(turns_lo, turns_hi) for _ in range(sessions)]
    for turn in range(max(turns)):
        for s in range(sessions):
            if turn >= turns[s]:
                continue
            t += rng.expovariate(rate)
            n_in = int(min(input_cap, max(1, rng.lognormvariate(math.log(median_input), sigma))))
            n_out = rng.randint(out_lo, out_hi)
            histories[s] = histories[s] + [rng.randrange(vocab) for _ in range(n_in)]
            reqs.append(dict(rid=rid, session=s, arrival=t, prompt=list(histories[s]), max_new=n_out))
            # the reply becomes part of the next turn's history (token values are irrelevant to the cache)
            histories[s] = histories[s] + [rng.randrange(vocab) for _ in range(n_out)]
            rid += 1
    return reqs


import os as _os

_os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")      # stdout carries the result line only


def main():
    import torch
    from ..models.dsa_moe import DsaMoeConfig
    from ..serving.server import ServingEngine

    ap = argparse.ArgumentParser()
    ap.add_argument("--sessions", type=int, default=8)
    ap.add_argument("--turns", default="2,3")
    ap.add_argument("--system-prefix", type=int, default=512)
    ap.add_argument("--median-input", type=int, default=256)
    ap.add_argument("--sigma", type=float, default=0.8)
    ap.add_argument("--input-cap", type=int, default=2048)
    ap.add_argument("--output", default="16,32")
    ap.add_argument("--rate", type=float, default=4.0, help="request arrivals per second (Poisson)")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tiny", action="store_true", help="the small test model instead of the full-width one")
    ap.add_argument("--max-batch", type=int, default=16)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--device-records", type=int, default=32768)
    ap.add_argument("--host-multiple", type=float, default=2.0, help="host tier size as a multiple of the device tier")
    ap.add_argument("--workload", default="", help="replay a frozen workload file (experiments/workloads.py) instead of a generated trace")
    ap.add_argument("--workload-sha256", default=None, help="refuse the workload unless its payload has this hash")
    ap.add_argument("--workload-limit", type=int, default=0, help="serve only the first N requests of the workload")
    ap.add_argument("--ttft-prompt", type=int, default=0,
                    help="instead of the replay: time to first token of ONE request with this many prompt tokens")
    ap.add_argument("--sections", type=int, default=0,
                    help="with --ttft-prompt: also print the per-section device time of this chunk (0 = off)")
    ap.add_argument("--unique-layers", type=int, default=4, help="distinct layer weight sets kept resident (cycled)")
    args = ap.parse_args()
    if args.ttft_prompt:
        return ttft(args)
    cfg = DsaMoeConfig().tiny(layers=args.layers, topk=256) if args.tiny else DsaMoeConfig(layers=args.layers, unique_layer_weights=min(args.layers, 4))
    tl, th = (int(x) for x in args.turns.split(","))
    ol, oh = (int(x) for x in args.output.split(","))
    workload_hash = None
    if args.workload:
        from .workloads import as_trace, load_workload

        wl = load_workload(args.workload, args.workload_sha256)
        workload_hash = wl["manifest"]["payload_sha256"]
        trace = as_trace(wl, vocab=cfg.vocab, limit=args.workload_limit or None)
    else:
        trace = build_trace(sessions=args.sessions, turns_lo=tl, turns_hi=th, system_prefix=args.system_prefix,
                            median_input=args.median_input, sigma=args.sigma, input_cap=args.input_cap, out_lo=ol, out_hi=oh,
                            rate=args.rate, vocab=cfg.vocab)
    longest = max(len(r["prompt"]) + r["max_new"] for r in trace)
    import os
    import time

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, group, cpu_group = 0, None, None
    device = None
    if world > 1:
        # one process per GPU: every rank builds the same trace and serves the sessions dealt to it
        from ..serving.engine import init_distributed

        rank, world, local, group, cpu_group = init_distributed()
        device = torch.device("cuda", local)
        torch.cuda.set_device(device)
    srv = ServingEngine(cfg, max_batch=args.max_batch, max_context=longest + 64, device_records=args.device_records,
                        host_records=int(args.device_records * args.host_multiple), prefill_chunk=args.prefill_chunk,
                        device=device, rank=rank, world=world, group=group, cpu_group=cpu_group)
    mine = [r for r in trace if r["session"] % world == rank]
    if world > 1:
        import torch.distributed as dist

        dist.barrier(group=cpu_group)
    t0 = time.perf_counter()
    srv.clock = lambda: time.perf_counter() - t0
    for r in mine:
        srv.submit(r["rid"], r["prompt"], r["max_new"], r["arrival"])
    steps = 0
    while True:
        state = srv.step()
        if state == "done":
            break
        if state == "idle":
            time.sleep(0.001)
        steps += 1
    torch.cuda.synchronize()
    rep = srv.report()
    if world > 1:
        # percentiles over every rank's finished requests; counters summed
        fin = [r for r in srv.finished if r.first_token_time is not None]
        local_stats = dict(ttft=[r.first_token_time - r.arrival for r in fin],
                           tpot=[(r.finish_time - r.first_token_time) / max(1, len(r.generated) - 1) for r in fin if len(r.generated) > 1],
                           out_tokens=sum(len(r.generated) for r in fin), last_finish=max((r.finish_time for r in fin), default=0.0),
                           report=rep)
        every = [None] * world
        dist.all_gather_object(every, local_stats, group=cpu_group)
        from ..serving.server import percentile

        ttft_all = [t for e in every for t in e["ttft"]]
        tpot_all = [t for e in every for t in e["tpot"]]
        wall = max(e["last_finish"] for e in every) or 1e-9
        rep = {k: sum(e["report"][k] for e in every) for k in
               ("admitted_requests", "finished_requests", "rejected_requests", "prefill_tokens", "reused_prefix_tokens",
                "cached_prefix_pages", "kv_token_capacity", "promotions", "evictions", "unserved")}
        rep.update(ttft_s_p50=percentile(ttft_all, 50), ttft_s_p99=percentile(ttft_all, 99),
                   tpot_s_p50=percentile(tpot_all, 50), tpot_s_p99=percentile(tpot_all, 99),
                   output_tokens_per_s=sum(e["out_tokens"] for e in every) / wall,
                   decode_steps=max(e["report"]["decode_steps"] for e in every), ranks=world,
                   padding_steps_rank0=srv.stats.get("padding_steps", 0))
    if workload_hash is not None:
        rep["workload_sha256"] = workload_hash
    rep.update(experiment="online_serving", requests=len(trace), sessions=len({r["session"] for r in trace}), layers=cfg.layers,
               device_records=args.device_records, host_records=int(args.device_records * args.host_multiple),
               total_prompt_tokens=sum(len(r["prompt"]) for r in trace), engine_steps=steps)
    if rank == 0:
        print(json.dumps(rep))
    srv.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
