"""Snapshot as a KV bank, one GPU: fill -> save -> restore into a fresh engine -> decode both over a
common steady window and compare the tokens.

    python -m ulacache_b200.experiments.kv_bank --tiny --batch 4 --prompt-len 1000 --steps 8 --dir /tmp/bank

Phases and what is reported: ``fill_s`` (synthetic fill of the source engine), ``save_s`` / ``save_gb_per_s``
(quiescent save of every request's KV and index planes), ``restore_s`` / ``restore_gb_per_s`` (a second engine
with the same weights takes the snapshot: payload verified, records routed by directory, prefix tree
rebuilt), ``decode`` (both engines decode ``--steps`` tokens from the same inputs; ``tokens_equal`` says the
restored cache decodes exactly what the source does) and the steady-window tokens/s of each.

Reference: scripts/fill_kv.py, scripts/decode.py:105-665 (fill phase, snapshot, decode over a common steady
window), ulacache/tools/snapshot/cuda.py:53-649.
"""
from __future__ import annotations

import argparse
import json
import os
import time


def main(argv=None):
    import torch
    from ..models.dsa_moe import DsaMoeConfig
    from ..serving.engine import DecodeEngine
    from ..serving.radix_tree import RadixPrefixTree
    from ..tools.snapshot.bank import rebuild_prefix_tree, restore_routing
    from ..tools.snapshot.cache_io import read_index_records, restore, save_shard, write_index_records
    from ..tools.snapshot.format import SnapshotLayout, SnapshotReader, SnapshotRequest, finalize_snapshot

    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", required=True, help="snapshot directory (must not hold a committed snapshot)")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--owners", type=int, default=2, help="snapshot owner shards")
    args = ap.parse_args(argv)
    os.environ["ULC_DETERMINISTIC"] = "1"
    cfg = (DsaMoeConfig().tiny(layers=args.layers, topk=256) if args.tiny
           else DsaMoeConfig(layers=args.layers, unique_layer_weights=min(args.layers, 4)))

    def engine():
        return DecodeEngine(cfg, batch=args.batch, prompt_len=args.prompt_len, max_new_tokens=args.steps + 8, mode="dpa",
                            use_graph=False)

    src = engine()
    t0 = time.perf_counter()
    src.fill_synthetic()
    torch.cuda.synchronize()
    fill_s = time.perf_counter() - t0
    first_tokens = src.batch.tokens.clone()
    g = torch.Generator().manual_seed(0)
    requests = [SnapshotRequest(f"req{b}", torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist(),
                                [int(first_tokens[b])]) for b in range(args.batch)]
    ids = {r.key: src.request_ids[b] for b, r in enumerate(requests)}
    plane = src.cache.cache_specification.storage_layout.record_planes[0]
    layout = SnapshotLayout(model_fingerprint="dsa-moe-synthetic", owners=args.owners, layers=cfg.cache_layers,
                            mla_row_bytes=plane.bytes_per_record, index_anchors=tuple(range(cfg.cache_layers)),
                            kv_format=plane.native_encoding)
    t0 = time.perf_counter()
    for owner in range(args.owners):
        save_shard(src.cache, args.dir, layout, requests, ids, owner,
                   index_reader=lambda layer, rows: read_index_records(src.index_pool[layer], rows))
    finalize_snapshot(args.dir)
    save_s = time.perf_counter() - t0
    nbytes = args.batch * args.prompt_len * cfg.cache_layers * (plane.bytes_per_record + 132)
    # ---- restore into a fresh engine (same weights: same seed) ----
    dst = engine()
    new_ids = {}
    span = 64
    for b, r in enumerate(requests):
        rows = dst.cache.alloc(dst.geometry.tokens_per_request)
        dst.batch.req_pages[b] = (rows.view(-1, span)[:, 0] // span).to(torch.int32)
        new_ids[r.key] = rows[: args.prompt_len]
    dst.request_ids = [new_ids[r.key] for r in requests]
    dst.batch.lengths.fill_(args.prompt_len)
    dst.batch.tokens.copy_(first_tokens)
    routing = restore_routing(args.owners, [r.key for r in requests], world=1, mode="dpa")
    t0 = time.perf_counter()
    written = restore(dst.cache, args.dir, new_ids,
                      index_writer=lambda layer, rows, data: write_index_records(dst.index_pool[layer], rows, data))
    torch.cuda.synchronize()
    restore_s = time.perf_counter() - t0
    tree = RadixPrefixTree()
    dup = rebuild_prefix_tree(tree, SnapshotReader(args.dir).requests,
                              {r.key: (new_ids[r.key][::64] // 64).tolist() for r in requests})
    # ---- decode both over the same window ----
    out = {}
    for name, eng in (("source", src), ("restored", dst)):
        toks = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            toks.append(eng.step_device().clone())
        torch.cuda.synchronize()
        out[name] = (torch.stack(toks), args.batch * args.steps / (time.perf_counter() - t0))
        eng.check()
    rep = dict(experiment="kv_bank", model="tiny" if args.tiny else "full width", layers=cfg.layers, batch=args.batch,
               prompt_len=args.prompt_len, snapshot_owners=args.owners, shards_read_by_rank0=len(routing[0]),
               snapshot_bytes=nbytes, fill_s=round(fill_s, 3), save_s=round(save_s, 3),
               save_gb_per_s=round(nbytes / save_s / 1e9, 3), restore_s=round(restore_s, 3),
               restore_gb_per_s=round(nbytes / restore_s / 1e9, 3), records_written=int(written),
               prefix_pages_cached=tree.cached_pages(), duplicate_pages=sum(dup.values()),
               tokens_equal=bool(torch.equal(out["source"][0], out["restored"][0])),
               decode_tokens_per_s=dict(source=round(out["source"][1], 1), restored=round(out["restored"][1], 1)))
    print(json.dumps(rep))
    src.close()
    dst.close()
    return 0 if rep["tokens_equal"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
