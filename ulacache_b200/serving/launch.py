"""One launcher for every decode method (run under torchrun for more than one GPU):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m ulacache_b200.serving.launch --method ulacache --mode dpa --phase decode --batch-per-gpu 32

Methods (what the KV cache looks like; the model, kernels and timing are the same for all):

* ``ulacache``  the pooled cache: ``--mode dpa`` keeps each request's records on its own rank with a host
  tier underneath; ``--mode tp`` stores every record once, striped over the ranks by 64-token page.
* ``hicache``   the replicated baseline: tensor-parallel heads, every rank keeps ALL records and index keys
  (KV capacity of one GPU), a host tier underneath with the same recency policy.
* ``hisparse``  the hot-buffer baseline: replicated KV whose device tier is only ``--hot-buffer`` records
  per request (twice the top-k by default); everything else lives in pinned host memory and is fetched
  on selection.

Phases: ``decode`` fills the cache synthetically, captures the step and reports tokens/s over a steady
window; ``fill`` stops after the fill and reports capacity and fill time; ``capacity`` prints what the
method admits under the byte budget without touching a GPU; ``--dry-run`` prints the resolved engine
arguments.

Reference: scripts/7_2_throughput/start_ulacache.sh, start_baseline.sh, start_hisparse.sh (one launcher per
method with --mode / --phase / --dry-run), scripts/decode.py:105-665 (fill and decode phases).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

METHODS = ("ulacache", "hicache", "hisparse")
RECORD_BYTES = 656 + 132          # KV record + index key, per token and layer


def resolve(args, world: int) -> dict:
    """Engine arguments of a method: layout, batch, device / host record capacities per rank."""
    from ..models.dsa_moe import DsaMoeConfig

    cfg_layers = args.layers or DsaMoeConfig().layers
    if args.method == "ulacache":
        mode, layout = args.mode, "pooled"
    else:
        mode, layout = "tp", "replicated"
    global_batch = args.batch_per_gpu * world
    batch = global_batch if mode == "tp" else args.batch_per_gpu
    kv_ranks = world if (mode == "tp" and layout == "pooled") else 1
    span = 64 * kv_ranks
    tokens = (args.prompt_len + args.max_new_tokens + 1 + span - 1) // span * span
    needed = (batch * tokens // kv_ranks + 64 + 63) // 64 * 64        # as the engine counts them
    device = host = None
    if args.method == "hisparse":
        device = max(64, batch * args.hot_buffer // 64 * 64)
        host = max(0, needed - device) + 64
    elif args.host_fraction > 0:
        device = max(64, int(needed * (1.0 - args.host_fraction)) // 64 * 64)
        host = needed - device + 64
    return dict(method=args.method, mode=mode, kv_layout=layout, world=world, global_batch=global_batch,
                batch_per_engine=batch, prompt_len=args.prompt_len, max_new_tokens=args.max_new_tokens,
                layers=cfg_layers, records_per_rank=needed, device_record_capacity=device, host_record_capacity=host or 0,
                kv_bytes_per_rank=needed * RECORD_BYTES * cfg_layers)


def capacity(args, world: int) -> dict:
    """Tokens a method admits per 8-GPU job under ``--kv-budget-hbm-gb`` + ``--kv-budget-host-gb`` per rank."""
    from ..models.dsa_moe import DsaMoeConfig

    layers = args.layers or DsaMoeConfig().layers
    per_token = RECORD_BYTES * layers
    hbm = int(args.kv_budget_hbm_gb * 2 ** 30) // per_token
    host = int(args.kv_budget_host_gb * 2 ** 30) // per_token
    if args.method == "ulacache":
        total = (hbm + host) * world                       # every record stored once
        device = hbm * world
    elif args.method == "hicache":
        total, device = hbm + host, hbm                    # every rank holds the same records
    else:
        total, device = host, hbm                          # the device tier is a cache of the host copy
    return dict(method=args.method, world=world, tokens_admitted=total, tokens_on_device=device,
                requests_of_prompt_len=total // max(1, args.prompt_len), budget_per_rank_gb=dict(hbm=args.kv_budget_hbm_gb,
                                                                                              host=args.kv_budget_host_gb))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--method", default="ulacache", choices=METHODS)
    ap.add_argument("--mode", default="dpa", choices=["tp", "dpa"], help="ulacache only: attention layout")
    ap.add_argument("--phase", default="decode", choices=["decode", "fill", "capacity"])
    ap.add_argument("--batch-per-gpu", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=32768)
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers for a quick look (marks the result invalid)")
    ap.add_argument("--unique-layers", type=int, default=0, help="distinct layer weight sets kept resident (0 = as many as fit)")
    ap.add_argument("--hot-buffer", type=int, default=4096, help="hisparse: device records per request")
    ap.add_argument("--host-fraction", type=float, default=0.0, help="ulacache / hicache: share of every context that starts in host memory")
    ap.add_argument("--kv-budget-hbm-gb", type=float, default=64.0)
    ap.add_argument("--kv-budget-host-gb", type=float, default=128.0)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    plan = resolve(args, world)
    if args.dry_run or args.phase == "capacity":
        out = capacity(args, world) if args.phase == "capacity" else plan
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(out))
        return 0
    import time

    import torch
    from ..models.dsa_moe import DsaMoeConfig
    from .engine import DecodeEngine, init_distributed

    # whatever NCCL logs (its version banner at the VERSION and WARN levels, more at INFO) goes to stderr:
    # stdout carries the result line only
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from bench import pick_unique_layers

    rank, world, local, group, cpu_group = init_distributed()
    cfg = DsaMoeConfig(layers=args.layers) if args.layers else DsaMoeConfig()
    budget = max(20.0, min(125.0, 150.0 - (plan["device_record_capacity"] or plan["records_per_rank"]) * RECORD_BYTES * cfg.layers / 1e9))
    unique = args.unique_layers or pick_unique_layers(cfg, world, budget * 1e9, plan["mode"])
    if unique < cfg.layers:
        cfg = DsaMoeConfig(layers=cfg.layers, unique_layer_weights=unique)
    eng = DecodeEngine(cfg, batch=plan["batch_per_engine"], prompt_len=args.prompt_len, max_new_tokens=args.max_new_tokens,
                       mode=plan["mode"], rank=rank, world=world, local_rank=local, group=group, cpu_group=cpu_group,
                       kv_layout=plan["kv_layout"], device_record_capacity=plan["device_record_capacity"],
                       host_record_capacity=plan["host_record_capacity"])
    t0 = time.perf_counter()
    eng.fill_synthetic()
    torch.cuda.synchronize()
    fill_s = time.perf_counter() - t0
    out = dict(plan, phase=args.phase, fill_s=round(fill_s, 2), distinct_layer_weight_sets_resident=unique,
               valid=not args.layers, memory=eng.memory_report())
    if args.phase == "decode":
        import torch.distributed as dist

        eng.warmup_and_capture()
        for _ in range(max(3, args.warmup)):
            eng.step_device()
        if world > 1:
            dist.barrier(group=group)
        torch.cuda.synchronize()
        before = eng.cache.counters() if plan["host_record_capacity"] else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            eng.step_device()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=eng.device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=group)
        eng.check()
        out.update(ms_per_step=round(float(ms) / args.steps, 3),
                   tokens_per_s=round(plan["global_batch"] * args.steps / (float(ms) / 1e3), 1))
        if before is not None:
            after = eng.cache.counters()
            d = {k: after[k] - before[k] for k in ("hits", "misses", "promotions", "evictions", "unserved")}
            out["host_tier"] = dict(promotions_per_step=d["promotions"] / args.steps, evictions_per_step=d["evictions"] / args.steps,
                                    hit_rate=round(d["hits"] / max(1, d["hits"] + d["misses"]), 4), unserved=d["unserved"],
                                    pcie_gb_per_s=round((d["promotions"] + d["evictions"]) * 656 / (float(ms) / 1e3) / 1e9, 2))
    if rank == 0:
        print(json.dumps(out))
    eng.close()
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
