"""KV capacity at a fixed memory budget: how many KV records (tokens) each cache organisation can
admit on 8 GPUs, for tensor-parallel attention (TP8) and data-parallel attention (DPA8), with and
without a speculative-decoding draft layer.

Three organisations are sized under the SAME per-rank budget (device bytes for KV + host bytes):

* ``replicated``  - every rank keeps the KV of every request it attends to in HBM (TP: all ranks hold
  the same tokens, so unique capacity is ONE rank's; DPA: ranks hold different requests).
* ``hot_buffer``  - the full KV lives in host memory, HBM holds a fixed hot buffer per request
  (TP: the host copy is replicated on every rank as well).
* ``pooled``      - this framework: every record is stored once, striped over all ranks' HBM and host
  tiers; the index stays in HBM; capacity planned by ``storage.capacity.plan_cache_capacity``.

With ``--audit-dir`` the per-rank start-up receipts ``rank*.json`` written by the serving entry point
are summed instead (what a running deployment actually allocated).

Reference: scripts/7_4_capacity/run.py:1-100 and README.md:32-35 (the table this reproduces).
"""
from __future__ import annotations

import argparse
import glob
import json
import os

from ..storage.capacity import CacheMemoryBudget, plan_cache_capacity, simple_usage_model

RECORD_BYTES = 656
INDEX_BYTES_PER_TOKEN = 132


def organisations(*, device_gb: float, host_gb: float, ranks: int, layers: int, requests_per_rank: int,
                  hot_records: int = 4096):
    dev, host = int(device_gb * 1e9), int(host_gb * 1e9)
    per_token_full = layers * (RECORD_BYTES + INDEX_BYTES_PER_TOKEN)
    out = {}
    # replicated: HBM only bounds it (a write-through host copy adds nothing to what can be attended)
    rep = dev // per_token_full
    out["replicated"] = {"tp": rep, "dpa": rep * ranks}
    # hot buffer: host holds payload, HBM holds index of every token + hot buffers
    hot_hbm = requests_per_rank * hot_records * layers * RECORD_BYTES
    by_host = host // (layers * RECORD_BYTES)
    by_index = max(0, dev - hot_hbm) // (layers * INDEX_BYTES_PER_TOKEN)
    hb = min(by_host, by_index)
    out["hot_buffer"] = {"tp": hb, "dpa": hb * ranks}
    # pooled
    measure = simple_usage_model(record_bytes=RECORD_BYTES, layers=layers, index_layers=layers, metadata_groups=layers)
    plan = plan_cache_capacity(memory_budget=CacheMemoryBudget(dev, host), measure_memory_usage=measure,
                               minimum_device_token_capacity=64 * 64, maximum_token_capacity_per_owner=1 << 28,
                               storage_owner_count=ranks)
    pooled = plan.usable_history_token_capacity()
    out["pooled"] = {"tp": pooled, "dpa": pooled,
                     "device_tokens_per_rank": plan.device_token_capacity_per_owner,
                     "host_tokens_per_rank": plan.host_token_capacity_per_owner}
    return out


def history_audit(*, device_gb: float, host_gb: float, ranks: int, layers: int, requests: int, max_context: int) -> dict:
    """The pooled organisation as an addressable-history audit: one request namespace, one KV partition whose owners
    are the ranks' planned tiers, bounded by the allocator (what was planned) and by request addressing."""
    from ..storage.capacity import (RecordOwnerCapacity, RequestNamespaceCapacityBounds, RequiredCachePartitionCapacity,
                                    addressable_tokens_per_owner, calculate_addressable_history_capacity)
    from ..storage.layout import StorageLayout

    org = organisations(device_gb=device_gb, host_gb=host_gb, ranks=ranks, layers=layers, requests_per_rank=max(1, requests // ranks))
    dev, host = org["pooled"]["device_tokens_per_rank"], org["pooled"]["host_tokens_per_rank"]
    owners = tuple(RecordOwnerCapacity(r, dev, host) for r in range(ranks))
    part = RequiredCachePartitionCapacity(0, "kv", StorageLayout(name="mla.scaled656"), owners, reserved_logical_record_count=64 * ranks)
    addressable = addressable_tokens_per_owner(maximum_requests=requests, maximum_context_tokens=max_context, owners=ranks) * ranks
    bounds = RequestNamespaceCapacityBounds(0, (dev + host) * ranks, addressable)
    return calculate_addressable_history_capacity([part], [bounds])


def from_audit(directory: str):
    files = sorted(glob.glob(os.path.join(directory, "rank*.json")))
    if not files:
        raise SystemExit(f"no rank*.json receipts under {directory}")
    dev = host = 0
    for f in files:
        with open(f) as fh:
            r = json.load(fh)
        dev += int(r["device_record_capacity"])
        host += int(r.get("host_record_capacity", 0))
    return {"ranks": len(files), "device_records": dev, "host_records": host, "unique_kv_records": dev + host}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device-gb", type=float, default=72.0, help="HBM per rank left for KV + index after weights")
    ap.add_argument("--host-gb", type=float, default=128.0, help="pinned host memory per rank")
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--layers", type=int, default=61)
    ap.add_argument("--requests-per-rank", type=int, default=64)
    ap.add_argument("--audit-dir", default="")
    ap.add_argument("--history-audit", action="store_true",
                    help="print the pooled organisation as an addressable-history audit (partitions, owners, bounds)")
    ap.add_argument("--max-context", type=int, default=131072)
    args = ap.parse_args()
    if args.history_audit:
        print(json.dumps({"experiment": "capacity_history_audit",
                          **history_audit(device_gb=args.device_gb, host_gb=args.host_gb, ranks=args.ranks, layers=args.layers,
                                          requests=args.requests_per_rank * args.ranks, max_context=args.max_context)}))
        return
    if args.audit_dir:
        print(json.dumps({"experiment": "capacity_audit", **from_audit(args.audit_dir)}))
        return
    for spec_on in (False, True):
        layers = args.layers + (1 if spec_on else 0)          # the draft layer keeps KV of its own
        org = organisations(device_gb=args.device_gb, host_gb=args.host_gb, ranks=args.ranks, layers=layers,
                            requests_per_rank=args.requests_per_rank)
        for mode in ("tp", "dpa"):
            row = {"experiment": "capacity", "mode": f"{mode}{args.ranks}", "speculative": spec_on,
                   "device_gb_per_rank": args.device_gb, "host_gb_per_rank": args.host_gb,
                   "kv_records": {k: v[mode] for k, v in org.items()}}
            row["pooled_vs_replicated"] = round(org["pooled"][mode] / max(1, org["replicated"][mode]), 2)
            row["pooled_vs_hot_buffer"] = round(org["pooled"][mode] / max(1, org["hot_buffer"][mode]), 2)
            print(json.dumps(row))


if __name__ == "__main__":
    main()
