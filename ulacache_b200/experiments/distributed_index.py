"""Distributed Index micro-benchmark (one layer): index keys are fp8 (128 dims + one fp32 scale per
token), sharded by 64-token page over the ranks; queries are 64 indexer heads x 128 dims with
per-head weights, replicated on every rank; each request selects the top 2048 of its context.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m ulacache_b200.experiments.distributed_index --context 32768,65536,131072 --batch 1,16,64,256

Three arms, device time of a CUDA-graph replay, max over ranks:

* ``fused``     score the local shard (fp8 tcgen05; the rows' score histograms are built in the score
                kernel's epilogue) -> histogram-first radix select with the logical-id epilogue
                -> candidates peer-stored into every rank's merge buffer -> one flag barrier -> merge top-k;
* ``allgather`` score the local shard -> library all-gather of the fp32 score slices -> transpose to
                row-major -> top-k over the gathered row through a rank-major -> logical column table;
* ``lines``     as ``allgather`` with the barrier-free 128-byte-line all-gather instead of the library's.

Bytes that must cross NVLink per rank: fused = (ranks-1) * B * 2048 * 8; all-gather =
(ranks-1) * B * context/ranks * 4.  The roofline is the slower of the local score read
(B * context/ranks * 132 B over HBM) and the fused arm's NVLink bytes over 770 GB/s.

Reference: indexer/scorer.py:96-369 + FlashAG score all-gather + TopKRankMajorKernel (topk_v2.cuh:1467).
"""
from __future__ import annotations

import argparse

from ..benchmarks.common import NVLINK_GBS, emit, measured_peaks, time_cuda_graph


def main():
    import torch
    import torch.distributed as dist
    from ..indexer import IndexOwnership
    from ..ops import _native as N
    from ..ops import indexer, topk as topk_op
    from ..parallel.peer_collectives import PeerCandidateExchange
    from ..parallel.symmetric import SymmetricHeap
    from ..serving.engine import init_distributed

    ap = argparse.ArgumentParser()
    ap.add_argument("--context", default="32768,131072")
    ap.add_argument("--batch", default="1,16,64,256")
    ap.add_argument("--topk", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--lines", type=int, default=1, help="also time the line all-gather arm")
    ap.add_argument("--pool-pages", type=int, default=1 << 16, help="index pages per rank (8448 B each)")
    args = ap.parse_args()
    rank, world, local, group, cpu_group = init_distributed()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    contexts = [int(c) for c in args.context.split(",")]
    batches = [int(b) for b in args.batch.split(",")]
    bmax, k = max(batches), args.topk
    own = IndexOwnership(world, 64)
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    pool = torch.randint(0, 255, (args.pool_pages, 8448), dtype=torch.uint8, device=dev, generator=g)
    pool[:, :8192] &= 0x7E                                    # fp8 codes without NaNs, moderate magnitudes
    pool[:, 8192:].view(torch.float32).copy_(torch.rand(args.pool_pages, 64, device=dev, generator=g) * 0.02 + 0.01)
    from ..flashag import LineScoreAllGather, line_count

    line_bytes = sum(2 * world * line_count(b, (c + own.span - 1) // own.span * 64) * 128 + 4096
                     for c in contexts for b in batches) if args.lines else 0
    heap = SymmetricHeap(cpu_group=cpu_group, rank=rank, world_size=world,
                         nbytes=4 * world * bmax * k * 4 + line_bytes + (8 << 20), device=dev) if world > 1 else None
    cand = PeerCandidateExchange(heap, bmax, k) if world > 1 else None
    ws = topk_op.workspace(bmax, dev)
    status = N.new_status(dev)
    peaks = measured_peaks()

    def max_over_ranks(us):
        t = torch.tensor([us], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return float(t)

    qgen = torch.Generator(device=dev).manual_seed(99)        # queries are replicated
    for ctx in contexts:
        local_pages = (ctx + own.span - 1) // own.span
        cols = local_pages * 64
        for B in batches:
            if B * local_pages > args.pool_pages:
                continue
            q = torch.randn(B, 1, 64, 128, device=dev, generator=qgen)
            w = torch.rand(B, 1, 64, device=dev, generator=qgen)
            q8, wf = indexer.quantize_queries(q, w)
            pages = torch.randperm(args.pool_pages, device=dev, generator=g)[: B * local_pages].view(B, local_pages).to(torch.int32)
            lengths = torch.full((B,), ctx, dtype=torch.int32, device=dev)
            # rank-major -> logical column table for the all-gather arm
            table = own.logical_token(torch.arange(world, device=dev).unsqueeze(1),
                                      torch.arange(cols, device=dev).unsqueeze(0)).reshape(1, -1).to(torch.int32)
            table = table.expand(B, -1).contiguous()
            ident_pages = torch.arange(local_pages, device=dev, dtype=torch.int32).unsqueeze(0).expand(B, -1).contiguous()

            def fused():
                logits = indexer.index_score(q8, wf, pages, lengths, pool, ranks=world, rank=rank, status=status,
                                             topk_workspace=ws)
                ids, vals = indexer.select_topk(logits, k, ident_pages, n_q=1, ranks=world, rank=rank, with_values=True,
                                                hist_workspace=ws)
                if cand is None:
                    return ids
                cv, ci = cand.exchange(ids, vals)
                return topk_op.topk(cv, k, in_idx=ci)

            def allgather():
                logits = indexer.index_score(q8, wf, pages, lengths, pool, ranks=world, rank=rank, status=status)
                if world == 1:
                    return topk_op.topk(logits, k, xform=table)
                gathered = torch.empty((world, B, cols), dtype=torch.float32, device=dev)
                dist.all_gather_into_tensor(gathered, logits, group=group)
                rows = gathered.permute(1, 0, 2).reshape(B, world * cols).contiguous()
                return topk_op.topk(rows, k, xform=table)

            line = LineScoreAllGather(heap, B, cols, name=f"line_{ctx}_{B}", slots=2) if (world > 1 and args.lines) else None

            def lines():
                logits = indexer.index_score(q8, wf, pages, lengths, pool, ranks=world, rank=rank, status=status)
                gathered = line.all_gather_scores(logits)
                rows = gathered.permute(1, 0, 2).reshape(B, world * cols).contiguous()
                return topk_op.topk(rows, k, xform=table)

            a = fused()
            b = allgather()
            torch.cuda.synchronize()
            N.raise_on_status(status, "distributed index")
            same = all(set(x) == set(y) for x, y in zip(a.sort(dim=1).values.tolist()[:4], b.sort(dim=1).values.tolist()[:4]))
            us_f = max_over_ranks(time_cuda_graph(fused, iters=args.iters))
            us_a = max_over_ranks(time_cuda_graph(allgather, iters=args.iters))
            us_l = None
            if line is not None:
                c = lines()
                torch.cuda.synchronize()
                N.raise_on_status(heap.status, "line all-gather")
                same = same and bool(torch.equal(c.sort(dim=1).values[:4], b.sort(dim=1).values[:4]))
                us_l = round(max_over_ranks(time_cuda_graph(lines, iters=args.iters)), 1)
            read = B * local_pages * 8448
            nvl = (world - 1) * B * k * 8
            roof = max(read / (peaks["hbm_gbs"] * 1e3), nvl / (NVLINK_GBS * 1e3))
            if rank == 0:
                emit(kernel="indexer_score_topk_merge", ranks=world, context=ctx, batch=B, topk=k, fused_us=round(us_f, 1),
                     allgather_us=round(us_a, 1), lines_us=us_l, speedup=round(us_a / us_f, 2), roofline_us=round(roof, 1),
                     fused_frac_of_roofline=round(roof / us_f, 3), same_selection_first_rows=bool(same),
                     nvlink_bytes_fused=nvl, nvlink_bytes_allgather=(world - 1) * B * cols * 4, peak=peaks["source"])
    if heap is not None:
        heap.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
