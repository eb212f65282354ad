"""Timing and roofline helpers shared by the micro-benchmarks."""
from __future__ import annotations

import json
import os

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
NVLINK_GBS = 770.0          # measured peer copy, per direction per GPU


def measured_peaks():
    """Copy bandwidth and bf16 GEMM throughput measured on this pool (MEASURED_PEAKS.json at the
    repository root when present, the documented fallback otherwise)."""
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS)


def time_cuda(fn, *, warmup=3, iters=10):
    """Microseconds per call: CUDA events around ``iters`` back-to-back calls after ``warmup``
    calls, with a synchronize on both sides.  Nothing but ``fn`` runs inside the timed region,
    so callers rotate over inputs larger than L2 instead of flushing it."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3        # microseconds per call


def time_cuda_graph(fn, *, warmup=2, iters=12, replays=3):
    """Microseconds of DEVICE time per call: ``iters`` calls are captured into one CUDA graph and the
    graph is replayed, so host launch cost (which exceeds the device time of small kernels) does not
    count.  ``fn`` must be capture-safe (no synchronisation; it may allocate through torch)."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for _ in range(iters):
            fn()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * replays) * 1e3


def emit(**kw):
    print(json.dumps(kw), flush=True)
