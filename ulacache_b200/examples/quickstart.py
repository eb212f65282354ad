"""The five verbs of the cache on one device, end to end: a cache whose HBM tier is smaller than the history, so
that reads promote records from the host tier and evict others.

    python -m ulacache_b200.examples.quickstart --device cpu     # or cuda

Reference: README.md "Minimal API" of the reference (init / alloc / write / access / free).
"""
from __future__ import annotations

import argparse
import json


def run(device: str = "cpu", *, layers: int = 2, tokens: int = 1000, device_pages: int = 4, host_pages: int = 16,
        queries: int = 2, topk: int = 128, steps: int = 4) -> dict:
    import torch

    import ulacache_b200 as ula
    from ulacache_b200.ops import records

    spec = ula.UnifiedCacheSpecification(
        storage_layout=ula.KeyValueStorageLayout(),                               # one plane of 656-byte fp8 MLA records
        layer_reuse=ula.LayerReuseSpecification.independent(layers),              # every layer selects for itself
        sparse_access=ula.SparseAccessSpecification(queries, topk),
        capacity_plan=ula.MemoryTierCapacity(device_record_capacity=device_pages * 64, host_record_capacity=host_pages * 64,
                                             maximum_write_record_count=8192,
                                             maximum_residency_input_record_count=min(device_pages * 64, queries * (topk + 1))))
    cache = ula.init(spec, ula.LocalCacheBindings(device=device))
    g = torch.Generator().manual_seed(0)
    latent = torch.randn(tokens, 512, generator=g).to(device)
    rope = torch.randn(tokens, 64, generator=g).to(device)

    ids = cache.alloc(tokens)                                                     # logical ids; HBM first, then host slots
    for layer in range(layers):
        cache.write(ids, layer, (latent * (layer + 1), rope))                     # quantised to fp8 records by the writer
    exact = 0
    for step in range(steps):
        pick = torch.stack([torch.randperm(tokens, generator=g)[:topk] for _ in range(queries)]).to(device)
        cache.begin_model_forward()
        for layer in range(layers):
            view = cache.access(ids[pick], layer)                                 # residency transaction + resolved locations
            assert bool((view.device_record_indices >= 0).all())                  # everything selected is now in HBM
            got = records.decode_scaled656(cache.gather_selected_records(layer))
            want = records.decode_scaled656(records.encode_scaled656(latent * (layer + 1), rope))[pick.reshape(-1)]
            exact += int((got == want).all(dim=1).sum())
            cache.finish_layer_attention(layer)
        cache.finish_model_forward()
    cache.check()
    out = dict(device=device, records=tokens, reads=steps * layers * queries * topk, reads_exact=exact, **cache.counters())
    cache.free(ids)
    cache.close()
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    print(json.dumps(run(ap.parse_args().device)))
