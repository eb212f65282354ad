"""Weight-streaming bandwidth of the block-scaled fp8 (grouped) GEMM at decode shapes.

    python -m ulacache_b200.benchmarks.fp8_gemm [--small]

Weights are rotated over several copies so every call reads HBM, not L2.  ``--small``
runs one short case (for profiler captures).
"""
from __future__ import annotations

import argparse

from .common import emit, measured_peaks, time_cuda, time_cuda_graph


def dense_sweep(args):
    """Input projection (7168 -> 2304), q_b + indexer q (1536 -> 32768) and o_proj (16384 -> 7168) with
    the row counts of decode; device time per launch (weights rotate over copies, so they come from HBM)."""
    import torch
    from ..ops import fp8

    dev = "cuda"
    peaks = measured_peaks()
    for (name, Nout, K) in [("w_in", 2304, 7168), ("w_qb", 32768, 1536), ("w_o", 7168, 16384)]:
        ws = [fp8.random_fp8_weight((Nout, K), device=dev) for _ in range(6)]
        for M in (32, 64):
            x8, sx = fp8.act_quant(torch.randn(M, K, device=dev, dtype=torch.bfloat16))
            for rows_hint in (16, 32, 64):
                if rows_hint > M:
                    continue
                for splits in sorted({1, 2, 4, 8, 16, fp8.pick_splits(Nout, K)}):
                    if splits > K // 128:
                        continue
                    i = [0]

                    def run():
                        q, s = ws[i[0] % 6]
                        i[0] += 1
                        fp8.grouped_gemm(x8, sx, q, s, splits=splits, max_rows=rows_hint)

                    us = time_cuda_graph(run, iters=12)
                    gbs = Nout * K / us / 1e3
                    emit(kernel="fp8_grouped_gemm", case=f"{name} {Nout}x{K}", M=M, rows_hint=rows_hint, splits=splits,
                         picked=splits == fp8.pick_splits(Nout, K), us=round(us, 1), gb_per_s=round(gbs, 1),
                         frac_of_hbm_peak=round(gbs / peaks["hbm_gbs"], 3))
        del ws


def prefill_sweep(args):
    """The GEMMs of one decoder layer at prefill chunk sizes (``--rows`` tokens): the token-major kernel against
    the weight-stationary decode kernel; TFLOP/s of device time (inputs and weights exceed L2 for the MoE cases,
    the dense weights rotate over copies)."""
    import torch
    from ..ops import fp8

    dev = "cuda"
    peaks = measured_peaks()
    M = args.rows
    cases = [("w_in", 1, 2304, 7168, M), ("w_qb", 1, 32768, 1536, M), ("w_o", 1, 7168, 16384, M),
             ("moe_w13", 256, 4096, 7168, 8 * M), ("moe_w2", 256, 7168, 2048, 8 * M)]
    if args.small:
        cases = [("w_in", 1, 2304, 7168, M), ("moe_w13", 32, 4096, 7168, 8 * M)]
    for name, E, Nout, K, rows in cases:
        copies = 1 if E > 1 else 3
        ws = [fp8.random_fp8_weight((E, Nout, K) if E > 1 else (Nout, K), device=dev) for _ in range(copies)]
        x8, sx = fp8.act_quant(torch.randn(rows, K, device=dev, dtype=torch.bfloat16))
        offs = None
        if E > 1:                      # uniform routing: rows / E per expert, the remainder on the first experts
            counts = torch.full((E,), rows // E, dtype=torch.int64)
            counts[: rows % E] += 1
            offs = torch.zeros(E + 1, dtype=torch.int32)
            offs[1:] = counts.cumsum(0)
            offs = offs.to(dev)
        out = torch.empty((rows, Nout), dtype=torch.bfloat16, device=dev)
        i = [0]

        def token_major():
            q, s = ws[i[0] % copies]
            i[0] += 1
            fp8.many_rows_gemm(x8, sx, q, s, offs, out=out)

        def stationary():
            import os

            q, s = ws[i[0] % copies]
            i[0] += 1
            os.environ["ULC_PREFILL_GEMM"] = "0"
            fp8.grouped_gemm(x8, sx, q, s, offs, out=out, max_rows=128)
            os.environ["ULC_PREFILL_GEMM"] = "1"

        flops = 2.0 * rows * Nout * K
        for label, fn in (("token_major", token_major), ("weight_stationary", stationary)):
            us = time_cuda(fn, iters=args.iters, warmup=3)
            emit(kernel="fp8_gemm_prefill", arm=label, case=f"{name} E={E} {Nout}x{K}", rows=rows, us=round(us, 1),
                 tflops=round(flops / us / 1e6, 1), weight_gb_per_s=round(E * Nout * K / us / 1e3, 1),
                 frac_of_bf16_peak=round(flops / us / 1e6 / peaks["bf16_tflops"], 3))
        del ws


def main():
    import torch
    from ..ops import fp8

    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--dense-sweep", action="store_true",
                    help="the dense projections of one decoder layer at 32 and 64 rows: every K split and ring geometry")
    ap.add_argument("--prefill", action="store_true",
                    help="one layer's GEMMs at a prefill chunk of --rows tokens: token-major against weight-stationary")
    ap.add_argument("--rows", type=int, default=2048)
    args = ap.parse_args()
    if args.dense_sweep:
        return dense_sweep(args)
    if args.prefill:
        return prefill_sweep(args)
    dev = "cuda"
    peaks = measured_peaks()
    torch.manual_seed(0)
    E, Nout, K = (32, 4096, 7168) if args.small else (256, 4096, 7168)
    copies = 1 if args.small else 3
    sets = [fp8.random_fp8_weight((E, Nout, K), device=dev) for _ in range(copies)]
    for B in ((16,) if args.small else (16, 64, 128)):
        scores = torch.rand(B, E, device=dev)
        tope = torch.topk(scores, min(8, E), dim=-1).indices.reshape(-1)
        order = torch.argsort(tope, stable=True)
        counts = torch.zeros(E + 1, dtype=torch.int64, device=dev)
        counts.index_add_(0, tope, torch.ones_like(tope))
        offs = torch.zeros(E + 1, dtype=torch.int32, device=dev)
        offs[1:] = counts[:E].cumsum(0)
        active = int((counts[:E] > 0).sum())
        x = torch.randn(tope.numel(), K, device=dev, dtype=torch.bfloat16)
        x8, sx = fp8.act_quant(x)
        i = [0]

        def run():
            q, s = sets[i[0] % copies]
            i[0] += 1
            fp8.grouped_gemm(x8, sx, q, s, offs, max_rows=16 if B <= 64 else 32)

        us = time_cuda(run, iters=3 if args.small else args.iters)
        gbs = active * Nout * K / us / 1e3
        emit(kernel="fp8_grouped_gemm", case=f"moe_w13 E={E} B={B} active={active}", us=round(us, 1),
             gb_per_s=round(gbs, 1), frac_of_hbm_peak=round(gbs / peaks["hbm_gbs"], 3), peak=peaks["source"])
    del sets
    if args.small:
        return
    for (Nout, K, M, splits) in [(36864, 7168, 16, 1), (7168, 18432, 16, 2), (7168, 16384, 16, 2), (32768, 1536, 16, 1),
                                 (129280 // 128 * 128, 7168, 16, 1)]:
        ws = [fp8.random_fp8_weight((Nout, K), device=dev) for _ in range(4)]
        x8, sx = fp8.act_quant(torch.randn(M, K, device=dev, dtype=torch.bfloat16))
        i = [0]

        def run():
            q, s = ws[i[0] % 4]
            i[0] += 1
            fp8.grouped_gemm(x8, sx, q, s, splits=splits, max_rows=M)

        us = time_cuda(run, iters=args.iters)
        gbs = Nout * K / us / 1e3
        emit(kernel="fp8_grouped_gemm", case=f"dense {Nout}x{K} M={M} splits={splits}", us=round(us, 1),
             gb_per_s=round(gbs, 1), frac_of_hbm_peak=round(gbs / peaks["hbm_gbs"], 3), peak=peaks["source"])
        del ws


if __name__ == "__main__":
    main()
