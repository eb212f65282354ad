"""Single entry point of a deployment: configuration JSON -> typed configuration -> cache specification
-> cache client, before any model weight is touched, plus the per-rank start-up receipt that the
capacity experiment sums.

    python -m ulacache_b200.serving.entry --config ulacache_b200/config/models/b200-native-dpa.json \
        --layers 61 --audit-dir /tmp/audit [--device cpu] [--scale 0.001]

(or ``ULACACHE_CONFIGURATION=<file>``).  Under torchrun every rank writes ``<audit-dir>/rank<r>.json``
with the capacities and bytes it really allocated; ``python -m ulacache_b200.experiments.capacity
--audit-dir <dir>`` adds them up.  ``--scale`` shrinks the configured capacities (for dry runs on a
machine that is not the deployment target).

Reference: patches/sglang.patch:5178-5349 (ulacache/entry.py: one entry point, JSON -> typed config ->
install bindings before the model loads), :7896 (matrix_startup_audit: per-rank storage receipts).
"""
from __future__ import annotations

import argparse
import json
import os


def specification_from_configuration(cfg, *, layers: int, max_queries: int = 64, topk: int = 2048, scale: float = 1.0,
                                     kv_format: str = "scaled656"):
    """Cache specification for a decoded :class:`ModelConfiguration` (capacities per owner)."""
    from ..cache.access import SparseAccessSpecification
    from ..cache.layers import LayerReuseSpecification
    from ..cache.specification import MemoryTierCapacity, UnifiedCacheSpecification
    from ..storage.layout import StorageLayout, record_plane

    if not cfg.enabled:
        raise ValueError("the native control arm does not use the pooled cache")
    if cfg.device_token_capacity_per_owner is None:
        raise ValueError(f"adapter {cfg.adapter} is sized by the serving arguments; pass capacities explicitly")
    page = 64
    dev = max(page, int(cfg.device_token_capacity_per_owner * scale) // page * page)
    host = int(cfg.host_token_capacity_per_owner * scale) // page * page
    opts = cfg.options
    write_max = getattr(opts, "maximum_write_record_count", 8192)
    fmt = getattr(opts, "native_kv_format", kv_format)
    return UnifiedCacheSpecification(
        storage_layout=StorageLayout(record_planes=(record_plane(fmt),)),
        layer_reuse=LayerReuseSpecification.independent(layers),
        sparse_access=SparseAccessSpecification(max_queries, topk),
        capacity_plan=MemoryTierCapacity(device_record_capacity=dev, host_record_capacity=host,
                                         maximum_write_record_count=write_max,
                                         maximum_residency_input_record_count=min(dev, max_queries * (topk + 1))))


def start(config_path=None, *, layers: int, device="cuda", audit_dir: str = "", scale: float = 1.0, max_queries: int = 64,
          topk: int = 2048):
    """Build the cache client for this rank and (optionally) write its start-up receipt."""
    from .. import client
    from ..bindings import LocalCacheBindings
    from ..config.model_configuration import launch_environment, load_model_configuration

    cfg = load_model_configuration(config_path)
    if cfg is None:
        raise SystemExit("no configuration: pass --config or set ULACACHE_CONFIGURATION")
    exports = launch_environment(cfg)               # refuses legacy variables and values that contradict the file
    rank = int(os.environ.get("RANK", "0"))
    spec = specification_from_configuration(cfg, layers=layers, max_queries=max_queries, topk=topk, scale=scale)
    cache = client.init(spec, LocalCacheBindings(device=device))
    inv = cache.memory_inventory()
    receipt = {"rank": rank, "adapter": cfg.adapter, "layers": layers, "scale": scale,
               "device_record_capacity": inv["device_record_capacity"], "host_record_capacity": inv["host_record_capacity"],
               "device_key_value_bytes": inv["device_key_value_bytes"], "host_key_value_bytes": inv["host_key_value_bytes"],
               "metadata_bytes": inv["metadata_bytes"], "launch_environment": exports}
    if audit_dir:
        os.makedirs(audit_dir, exist_ok=True)
        with open(os.path.join(audit_dir, f"rank{rank}.json"), "w") as f:
            json.dump(receipt, f)
    return cache, receipt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=None)
    ap.add_argument("--layers", type=int, default=61)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--audit-dir", default="")
    ap.add_argument("--scale", type=float, default=1.0)
    args = ap.parse_args()
    cache, receipt = start(args.config, layers=args.layers, device=args.device, audit_dir=args.audit_dir, scale=args.scale)
    os.environ.update(receipt["launch_environment"])    # workers spawned from this process inherit the same settings
    print(json.dumps(receipt))
    cache.close()


if __name__ == "__main__":
    main()
