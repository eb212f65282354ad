"""Bandwidth of the barrier-free score all-gathers against the library collective (torchrun, one rank
per GPU):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m ulacache_b200.benchmarks.flashag --out flashag.json

For every message size each arm gathers ``rows x cols`` fp32 per rank from every rank.  Time is CUDA
events around a CUDA-graph replay of ``iters`` calls, max over ranks; ``egress_gbs`` = payload bytes one rank
sends to its peers per second ((world - 1) x bytes per rank / time), ``wire_gbs`` adds the tag words.
The NVLink reference on this pool is a peer copy of 770 GB/s per direction per GPU.

Reference figure: about 700 GB/s unicast on B300 (ulacache/csrc/flashag/b300/ag_kernels_dynamic.cuh:95-107).
"""
from __future__ import annotations

import argparse
import json


def main(argv=None):
    import torch
    import torch.distributed as dist
    from ..flashag import LineScoreAllGather, TaggedScoreAllGather, line_count
    from ..ops import _native as N
    from ..parallel.symmetric import SymmetricHeap
    from ..serving.engine import init_distributed

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--max-mb", type=float, default=16.0, help="largest message per rank")
    ap.add_argument("--ctas", default="0", help="comma list of CTA limits for the line kernel (0 = one per SM)")
    args = ap.parse_args(argv)
    rank, world, local, group, cpu_group = init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    shapes = [(32, 512), (32, 4096), (128, 4096), (512, 4096), (2048, 2048)]
    shapes = [s for s in shapes if s[0] * s[1] * 4 <= args.max_mb * 2 ** 20]
    slots = 2
    cta_limits = [int(c) for c in args.ctas.split(",")]
    # the heap is a bump allocator: room for every arm's receive slab of every shape
    heap_bytes = 8 << 20
    for r, c in shapes:
        heap_bytes += len(cta_limits) * (slots * world * line_count(r, c) * 128 + 4096) + 4 * world * r * c * 8 + 4096
    heap = SymmetricHeap(cpu_group=cpu_group, rank=rank, world_size=world, nbytes=heap_bytes, device=dev)
    results = []

    def timed(fn):
        """Device time per call: ``iters`` calls captured in one CUDA graph (the Python launch path
        costs more than a small all-gather), replayed once untimed and once timed."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(device=dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(args.iters):
                    fn()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        graph.replay()
        torch.cuda.synchronize()
        dist.barrier(group=group)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t) * 1e3          # microseconds, max over ranks

    for rows, cols in shapes:
        x = torch.randn(rows, cols, device=dev) + rank
        ref = torch.empty((world, rows, cols), device=dev)
        dist.all_gather_into_tensor(ref, x, group=group)
        nbytes = rows * cols * 4
        row = dict(rows=rows, cols=cols, bytes_per_rank=nbytes, world=world)
        for ctas in cta_limits:
            line = LineScoreAllGather(heap, rows, cols, name=f"line_{rows}_{cols}_{ctas}", slots=slots, max_ctas=ctas)
            got = line.all_gather_scores(x)
            torch.cuda.synchronize()
            N.raise_on_status(heap.status, "line all-gather")
            key = "line" if ctas == 0 else f"line_ctas{ctas}"
            row[key + "_same"] = bool(torch.equal(got, ref))
            us = timed(lambda: line.all_gather_scores(x))
            row[key + "_us"] = round(us, 2)
            row[key + "_egress_gbs"] = round((world - 1) * nbytes / us / 1e3, 1)
            row[key + "_wire_gbs"] = round((world - 1) * nbytes * 32 / 31 / us / 1e3, 1)
        words = TaggedScoreAllGather(heap, rows, cols, name=f"words_{rows}_{cols}")
        got = words.all_gather_scores(x)
        torch.cuda.synchronize()
        row["words_same"] = bool(torch.equal(got, ref))
        us = timed(lambda: words.all_gather_scores(x))
        row["words_us"] = round(us, 2)
        row["words_egress_gbs"] = round((world - 1) * nbytes / us / 1e3, 1)
        us = timed(lambda: dist.all_gather_into_tensor(ref, x, group=group))
        row["nccl_us"] = round(us, 2)
        row["nccl_egress_gbs"] = round((world - 1) * nbytes / us / 1e3, 1)
        N.raise_on_status(heap.status, "all-gather arms")
        results.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(dict(world=world, iters=args.iters, timing="CUDA events around a graph replay of `iters` calls, max over ranks",
                           results=results), f, indent=1)
    heap.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
