"""Rank-local engine for data-parallel attention: exclusive HBM / host tiers, no peers.

Reference: UnifiedLocalResidency (ulacache/cache/local_cache.py:11).
"""
from __future__ import annotations

from ..storage.layout import OwnerMap
from .engine import CacheEngine


class UnifiedLocalResidency(CacheEngine):
    def __init__(self, spec, bindings):
        super().__init__(spec, device=bindings.device, owners=OwnerMap(1, 6), my_rank=0,
                         options=bindings.execution_options,
                         host_pool_factory=bindings.allocate_host_record_storage)

    def offload_prefill(self, ids):
        """Move freshly written prefill records to the host tier when the prefill
        was allowed to borrow more HBM than it may keep (reference:
        offload_prefill_rows, ulacache/csrc/cache/prefix.cuh:10).  Implemented as
        release + re-register on the host tier with a record copy in between."""
        import torch

        ids = ids.reshape(-1)
        for g, res in enumerate(self.residency):
            mine, local = res._owned_locals(ids.to(torch.int32))
            rows = local[mine].long()
            e = res.directory[rows]
            on_dev = e >= 0
            if not bool(on_dev.any()):
                continue
            src_slots = e[on_dev].long()
            move_ids = ids[mine][on_dev]
            if self.is_cuda:
                self._offload_rows_on_device(g, res, rows[on_dev], src_slots, move_ids)
                continue
            saved = {}
            for layer in self.groups.layers_of(g):
                for p, st in enumerate(self.storages):
                    saved[(layer, p)] = self.layer_plane(layer, p)[src_slots].clone()
            res.release(move_ids)
            res.register(move_ids, prefer_device=False)
            e2 = res.directory[rows[on_dev]]
            for (layer, p), data in saved.items():
                host_rows = e2 <= -2
                if bool(host_rows.any()):
                    self.layer_host_plane(layer, p)[(-e2[host_rows] - 2).long().cpu()] = data[host_rows].cpu()
                dev_rows = e2 >= 0
                if bool(dev_rows.any()):
                    self.layer_plane(layer, p)[e2[dev_rows].long()] = data[dev_rows]

    def _offload_rows_on_device(self, g, res, rows, src_slots, move_ids):
        """CUDA path: the directory moves the rows to the host tier (release + register), then ONE copy
        kernel per layer and plane stores their records from the freed HBM slots into the pinned host
        planes (warp per record, 16-byte vectors, no staging through host tensors).  A freed slot keeps
        its bytes until something is written to it, and nothing is before the copies.  Rows that had to
        stay in HBM because the host tier is full (rare) move slot to slot through a device temporary."""
        import torch
        from ..ops import exchange as X

        res.release(move_ids)
        res.register(move_ids, prefer_device=False)
        e2 = res.directory[rows]
        to_host = e2 <= -2
        n_host = int(to_host.sum())
        src_h = src_slots[to_host].to(torch.int32).contiguous()
        dst_h = (-e2[to_host] - 2).to(torch.int32).contiguous()
        stay = e2 >= 0
        n_stay = int(stay.sum())
        for layer in self.groups.layers_of(g):
            for p, st in enumerate(self.storages):
                rb = st.plane.bytes_per_record
                plane = self.layer_plane(layer, p)
                if n_host:
                    X.copy_records(plane, src_h, self.layer_host_plane(layer, p).data_ptr(), dst_h, n_host, rb)
                if n_stay:
                    tmp = plane[src_slots[stay]]
                    plane[e2[stay].long()] = tmp
