"""Device time of the small per-layer kernels of a decode step at the headline shapes
(32 requests per GPU, 32K-token contexts, hidden 7168): top-k in both launch shapes, the
fused residual-add + RMSNorm + fp8 quantiser, the attention split merge, the SwiGLU
quantiser with and without the routed-row limit, and the batched per-head bf16 GEMMs.

    python -m ulacache_b200.benchmarks.decode_small_kernels [--topk-forms]

Each call is timed alone with CUDA events after a write of a 256 MB buffer (larger than
L2), so the inputs come from HBM as they do inside a step that streams expert weights
between two uses.  One JSON line per kernel.
"""
from __future__ import annotations

from .common import emit


def _time_flushed(fn, flush, *, warmup=5, iters=30):
    """Median microseconds of ``fn`` over ``iters`` calls, L2 flushed before each."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def topk_forms():
    """Every launch form of the stand-alone top-k over rows x context (k = 2048, normal scores): the cluster
    kernel, the histogram pair, and the one-CTA-per-row kernels (streaming and staged).  CUDA events around 8
    calls with a 256 MB write before each (its own time subtracted), one JSON line per shape."""
    import sys
    import torch
    from ..ops import topk
    from .common import time_cuda

    torch.manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    small = "--small" in sys.argv          # one shape (for profiler captures)
    for ctx in ((32768,) if small else (32768, 65536, 131072)):
        for rows in ((256,) if small else (8, 32, 64, 128, 256, 1024, 2048)):
            if rows * ctx * 4 > (1 << 30):
                continue
            x = torch.randn(rows, ctx, device="cuda")
            out = torch.empty(rows, 2048, dtype=torch.int32, device="cuda")
            base = time_cuda(lambda: flush.zero_(), iters=8)
            res = {}
            for name in ("auto", "cluster", "rows", "rows_staged"):
                topk.set_launch_mode(name)
                try:
                    res[name] = round(time_cuda(lambda: (flush.zero_(), topk.topk(x, 2048, out=out)), iters=8) - base, 1)
                finally:
                    topk.set_launch_mode("auto")
            res["hist"] = round(time_cuda(lambda: (flush.zero_(), topk.topk(x, 2048, out=out, method="hist")), iters=8) - base, 1)
            emit(kernel="topk_forms", rows=rows, length=ctx, k=2048, us=res)


def main():
    import sys
    import torch
    from ..ops import fp8, gemm, glue, topk
    from ..ops import prefill as P

    if "--topk-forms" in sys.argv:
        return topk_forms()
    dev = "cuda"
    torch.manual_seed(0)
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    rows, ctx, k = 32, 32768, 2048

    # ---- top-k: score distributions from wide (normal) to one coarse bin (what ReLU-weighted
    # index scores look like), both launch shapes, checked against the reference selection
    dists = {
        "normal": torch.randn(rows, ctx, device=dev),
        "one_octave": 4.0 + torch.rand(rows, ctx, device=dev),
        "relu_sum": torch.relu(torch.randn(rows, ctx, device=dev)) * 3 + torch.rand(rows, ctx, device=dev),
    }
    # sum over 64 indexer heads of weight * ReLU(q.k), built head by head to keep memory small
    acc = torch.zeros(rows, ctx, device=dev)
    for _ in range(64):
        acc += torch.relu(torch.randn(rows, ctx, device=dev)) * float(torch.rand(()))
    dists["index_like"] = acc
    for name, s in dists.items():
        ref = topk.topk_reference(s, k)
        for mode in ("row", "cluster"):
            topk.set_launch_mode(mode)
            try:
                out = topk.topk(s, k)
                torch.cuda.synchronize()
                same = all(sorted(out[r].tolist()) == sorted(ref[r].tolist()) for r in range(rows))
                us = _time_flushed(lambda: topk.topk(s, k), flush)
            finally:
                topk.set_launch_mode("auto")
            emit(kernel="topk", rows=rows, length=ctx, k=k, scores=name, launch=mode, us=round(us, 2),
                 matches_reference=same)
    for r in (8, 64, 128):
        s = torch.randn(r, ctx, device=dev)
        for mode in ("row", "cluster"):
            topk.set_launch_mode(mode)
            try:
                us = _time_flushed(lambda: topk.topk(s, k), flush)
            finally:
                topk.set_launch_mode("auto")
            emit(kernel="topk", rows=r, length=ctx, k=k, scores="normal", launch=mode, us=round(us, 2))

    # ---- residual add + RMSNorm + fp8 quantisation (1 partial and 8 partials)
    H = 7168
    x = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    d1 = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    d8 = torch.randn(8, rows, H, device=dev, dtype=torch.bfloat16)
    us = _time_flushed(lambda: glue.add_rmsnorm_quant(x, d1, w, 1e-6, want_h=True), flush)
    emit(kernel="add_rmsnorm_quant", rows=rows, hidden=H, partials=1, us=round(us, 2))
    us = _time_flushed(lambda: glue.add_rmsnorm_quant(x, d8, w, 1e-6, want_h=True, n_slots=8, slot_stride=rows * H),
                       flush)
    emit(kernel="add_rmsnorm_quant", rows=rows, hidden=H, partials=8, us=round(us, 2))

    # ---- merge of 4 KV splits for 32 queries x 128 heads
    po = torch.randn(4, rows * 128, 512, device=dev)
    pl = torch.randn(4, rows * 128, device=dev)
    us = _time_flushed(lambda: P.merge_partial_attention(po, pl), flush)
    emit(kernel="mla_combine", rows=rows * 128, splits=4, us=round(us, 2),
         gbs=round((po.numel() * 4 + rows * 128 * 512 * 2) / us / 1e3, 1))

    # ---- SwiGLU + quantise over a buffer sized for 256 tokens x 8 choices, 288 rows filled
    mid = torch.randn(2080, 4096, device=dev, dtype=torch.bfloat16)
    lim = torch.tensor([288], device=dev, dtype=torch.int32)
    q = torch.empty(2080, 2048, device=dev, dtype=torch.uint8)
    sc = torch.empty(2080, 16, device=dev)
    us = _time_flushed(lambda: fp8.act_quant(mid, swiglu=True, out_q=q, out_s=sc), flush)
    emit(kernel="act_quant_swiglu", rows=2080, limit=None, us=round(us, 2))
    us = _time_flushed(lambda: fp8.act_quant(mid, swiglu=True, out_q=q, out_s=sc, row_limit=lim), flush)
    emit(kernel="act_quant_swiglu", rows=2080, limit=288, us=round(us, 2))

    # ---- batched per-head bf16 projections around the attention kernel (128 heads)
    heads = 128
    qn = torch.randn(rows, heads, 128, device=dev, dtype=torch.bfloat16)
    w_uk = torch.randn(heads, 512, 128, device=dev, dtype=torch.bfloat16)
    o = torch.randn(rows, heads, 512, device=dev, dtype=torch.bfloat16)
    w_uv = torch.randn(heads, 128, 512, device=dev, dtype=torch.bfloat16)
    q_lat = torch.empty(rows, heads, 512, device=dev, dtype=torch.bfloat16)
    o_v = torch.empty(rows, heads, 128, device=dev, dtype=torch.bfloat16)
    us = _time_flushed(lambda: gemm.batched_linear(qn, w_uk, q_lat), flush)
    emit(kernel="gemm_wt_batched", what="q_nope x W_uk", heads=heads, n=512, k=128, us=round(us, 2),
         gbs=round(w_uk.numel() * 2 / us / 1e3, 1))
    us = _time_flushed(lambda: gemm.batched_linear(o, w_uv, o_v), flush)
    emit(kernel="gemm_wt_batched", what="o x W_uv", heads=heads, n=128, k=512, us=round(us, 2),
         gbs=round(w_uv.numel() * 2 / us / 1e3, 1))
    wr = torch.randn(256, H, device=dev, dtype=torch.bfloat16)
    hx = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
    us = _time_flushed(lambda: gemm.linear(hx, wr, splits=0), flush)
    emit(kernel="gemm_wt", what="router", n=256, k=H, us=round(us, 2))


if __name__ == "__main__":
    main()
