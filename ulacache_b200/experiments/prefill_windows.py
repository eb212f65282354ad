"""The two-window prefill pipeline at full window size (1,048,576 records per window) on one GPU.

    python -m ulacache_b200.experiments.prefill_windows [--records 1310720] [--queries 2048] [--topk 2048] [--layers 4]

A cache holds ``records`` encoded KV records per layer.  A prefill chunk of ``queries`` rows selects ``topk``
records each out of a range chosen so that the union fills most of a window.  Per layer the pipeline builds the
union (``selection_union`` kernel: flag / scan / scatter over the id space), gathers the union's records through the
directory into a window without touching residency state (``gather_by_directory``), and hands attention the
selection rewritten as window rows; the window of layer l + 1 fills on a side stream while a stand-in for the
attention of layer l (a bf16 GEMM of about the same duration) runs.  Reported: union time, fill time and bytes per
second against the measured copy rate, and the time of the whole layer loop with and without the overlap.

Reference: ulacache/transfer/prefill_pipeline.py:115-330 (LayerPrefillPipeline), cache/prefill/buffers.py:40-81
(two 1,048,576-record windows).
"""
from __future__ import annotations

import argparse
import json


def main():
    import torch
    import ulacache_b200 as ula
    from ..benchmarks.common import measured_peaks, time_cuda
    from ..bindings import LocalCacheBindings
    from ..cache.access import SparseAccessSpecification
    from ..cache.layers import LayerReuseSpecification
    from ..cache.prefill import PrefillWindowPair, ReadOnlyPrefillReader, SelectionWindowMap, WindowLeases
    from ..cache.prefill.buffers import DEFAULT_WINDOW_RECORDS
    from ..cache.specification import MemoryTierCapacity, UnifiedCacheSpecification
    from ..storage.layout import MLA_SCALED656, StorageLayout
    from ..transfer.prefill_pipeline import LayerPrefillPipeline

    ap = argparse.ArgumentParser()
    ap.add_argument("--records", type=int, default=1310720)
    ap.add_argument("--queries", type=int, default=2048)
    ap.add_argument("--topk", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--window", type=int, default=DEFAULT_WINDOW_RECORDS)
    ap.add_argument("--out", default="")
    ap.add_argument("--device", default="cuda")
    args = ap.parse_args()
    dev = args.device
    torch.manual_seed(0)
    spec = UnifiedCacheSpecification(
        storage_layout=StorageLayout(record_planes=(MLA_SCALED656,)),
        layer_reuse=LayerReuseSpecification.independent(args.layers),
        sparse_access=SparseAccessSpecification(args.queries, args.topk),
        capacity_plan=MemoryTierCapacity(device_record_capacity=args.records, host_record_capacity=0,
                                         maximum_write_record_count=1 << 16,
                                         maximum_residency_input_record_count=args.records))
    cache = ula.init(spec, LocalCacheBindings(device=dev))
    engine = cache.engine if hasattr(cache, "engine") else cache
    n_rec = args.records - 128                           # (the allocator keeps its first page)
    ids = cache.alloc(n_rec)
    rb = engine.layer_plane(0).shape[-1]
    for layer in range(args.layers):                      # encoded records, written in slices
        for a in range(0, n_rec, 1 << 16):
            part = ids[a:a + (1 << 16)]
            cache.write(part.to(dev), layer, torch.randint(0, 255, (part.numel(), rb), dtype=torch.uint8, device=dev))
    # a chunk's selection: ids drawn from a range slightly smaller than the window
    span = min(n_rec, int(args.window * 0.98))
    pick = torch.randint(0, span, (args.queries, args.topk), device=dev)
    sel = ids.to(dev)[pick].to(torch.int32)
    id_space = int(ids.max()) + 1
    wmap = SelectionWindowMap(id_space, args.window)
    pair = PrefillWindowPair(args.window, rb, dev)
    reader = ReadOnlyPrefillReader(engine)
    uni, count, rows = wmap.build(sel)
    n_union = int(count)
    # correctness on a sample: window rows hold the records the selection names
    missing = reader.fill(pair.current, 0, uni, count)
    if dev != "cpu":
        torch.cuda.synchronize()
    probe = torch.randint(0, args.queries * args.topk, (4096,), device=dev)
    want = engine.read_records(0, sel.reshape(-1)[probe])[0]
    same = bool(torch.equal(pair.current.data[rows.reshape(-1)[probe].long()], want)) and int(missing) == 0
    peaks = measured_peaks()
    union_us = time_cuda(lambda: wmap.build(sel), iters=5)
    fill_us = time_cuda(lambda: reader.fill(pair.current, 0, uni, count), iters=5)
    fill_bytes = 2.0 * n_union * rb                       # read from the pool, written to the window
    # stand-in for the attention of one layer: a bf16 GEMM sized to about the fill time
    m = 4096
    a16 = torch.randn(m, m, device=dev, dtype=torch.bfloat16)
    b16 = torch.randn(m, m, device=dev, dtype=torch.bfloat16)
    gemm_us = time_cuda(lambda: torch.matmul(a16, b16), iters=5)
    reps = max(1, round(fill_us / gemm_us))

    def attention():
        for _ in range(reps):
            torch.matmul(a16, b16)

    def loop(side):
        pipe = LayerPrefillPipeline(reader, wmap, pair, WindowLeases(), side_stream=side)
        pipe.prime(0, sel)
        for layer in range(args.layers):
            window, wrows = pipe.acquire(layer)
            if layer + 1 < args.layers:
                pipe.prefetch(layer + 1, sel)
            attention()
            pipe.release(layer)

    serial_us = time_cuda(lambda: loop(None), iters=3, warmup=1)
    side = torch.cuda.Stream() if dev != "cpu" else None
    overlap_us = time_cuda(lambda: loop(side), iters=3, warmup=1)
    res = dict(experiment="prefill_windows", records_per_layer=args.records, layers=args.layers, queries=args.queries,
               topk=args.topk, window_records=args.window, union_records=n_union, window_bytes=args.window * rb,
               rows_match_records=same, union_us=round(union_us, 1), fill_us=round(fill_us, 1),
               fill_gb_per_s=round(fill_bytes / fill_us / 1e3, 1),
               fill_fraction_of_copy_peak=round(fill_bytes / fill_us / 1e3 / peaks["hbm_gbs"], 3),
               attention_stand_in_us=round(gemm_us * reps, 1), layer_loop_serial_us=round(serial_us, 1),
               layer_loop_overlapped_us=round(overlap_us, 1),
               overlap_saving_fraction=round(1.0 - overlap_us / serial_us, 3), peaks=peaks.get("source", "fallback"))
    print(json.dumps(res), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(res, f, indent=1)
    cache.close()


if __name__ == "__main__":
    main()
