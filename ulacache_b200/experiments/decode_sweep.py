"""Decode throughput over batch sizes for one parallel layout (run under torchrun for N > 1):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m ulacache_b200.experiments.decode_sweep --mode dpa --batch-per-gpu 8,16,32

One JSON line per batch size: tokens/s, ms per step, KV records resident per rank.  Every point
builds a fresh engine (fill is part of set-up, not of the timed window), steps are CUDA-graph
replays timed with device events, max over ranks.

Reference: scripts/decode.py:105-665 (common steady window after a separate fill phase),
scripts/7_2_throughput/README.md (batch sweep to the largest admissible batch).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main():
    import torch
    from ..models.dsa_moe import DsaMoeConfig
    from ..serving.engine import DecodeEngine, init_distributed

    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="dpa", choices=["tp", "dpa"])
    ap.add_argument("--batch-per-gpu", default="8,16,32")
    ap.add_argument("--prompt-len", type=int, default=32768)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers for a quick look (not a valid benchmark)")
    ap.add_argument("--csv", default="", help="also append every point to this results.csv")
    args = ap.parse_args()
    # whatever NCCL logs (its version banner at the VERSION and WARN levels, more at INFO) goes to stderr:
    # stdout carries the result line only
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from bench import pick_unique_layers

    rank, world, local, group, cpu_group = init_distributed()
    for bpg in (int(b) for b in args.batch_per_gpu.split(",")):
        cfg = DsaMoeConfig(layers=args.layers) if args.layers else DsaMoeConfig()
        max_new = 2 * (args.warmup + args.steps) + 16
        pools = bpg * (args.prompt_len + max_new + 512) * (656 + 132) * cfg.layers
        budget = max(20.0, min(125.0, 152.0 - pools / 1e9))
        unique = pick_unique_layers(cfg, world, budget * 1e9, args.mode)
        if unique < cfg.layers:
            cfg = DsaMoeConfig(layers=cfg.layers, unique_layer_weights=unique)
        batch = bpg * world if args.mode == "tp" else bpg
        eng = DecodeEngine(cfg, batch=batch, prompt_len=args.prompt_len, max_new_tokens=max_new, mode=args.mode, rank=rank,
                           world=world, local_rank=local, group=group, cpu_group=cpu_group)
        torch.cuda.empty_cache()
        eng.fill_synthetic()
        torch.cuda.empty_cache()
        eng.warmup_and_capture()
        for _ in range(max(3, args.warmup)):
            eng.step_device()
        if world > 1:
            import torch.distributed as dist

            dist.barrier(group=group)
        torch.cuda.synchronize()
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
        mem = eng.memory_report()
        if rank == 0:
            gb = bpg * world
            row = {"experiment": "decode_sweep", "parallelism": f"{args.mode}{world}", "global_batch": gb,
                   "prompt_len": args.prompt_len, "ms_per_step": round(float(ms) / args.steps, 3),
                   "tokens_per_s": round(gb * args.steps / (float(ms) / 1e3), 1),
                   "kv_records_per_rank": mem["kv_records_per_rank"], "layers": cfg.layers,
                   "distinct_layer_weight_sets_resident": unique, "valid": not args.layers}
            print(json.dumps(row), flush=True)
            if args.csv:
                from ..utils import append_result_csv

                append_result_csv(args.csv, row)
        eng.close()
        del eng
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
