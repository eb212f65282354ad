"""Record-owner engine: disjoint owners in one namespace, consumers with
independent selections.

Consumers export their selections to the owners (all-gather of the padded
``[Q, K]`` ID tensors, or peer stores when a symmetric heap is bound); each owner
runs the residency transaction over the union of everybody's requests for rows it
owns; after the barrier every consumer resolves its own selection against the
owners' directories and reads the records from the owners' pools.

Reference: RecordOwnerPagedResidency (ulacache/cache/owner_cache.py:6: export
:323, gather :407, three-phase publication :457, agreement check via
all_gather_object :82-96).
"""
from __future__ import annotations

from .access import SparseAttentionAccessPlan
from .engine import CacheEngine, CollectiveTransport, P2PTransport


class RecordOwnerPagedResidency(CacheEngine):
    def __init__(self, spec, bindings):
        import torch

        device = torch.device(bindings.device)
        world, rank = bindings.world_size, bindings.rank
        self._group = bindings.owner_process_group
        heap = transport = None
        if world > 1:
            self._check_agreement(spec, bindings)
            if device.type == "cuda" and bindings.ipc_manager_factory is not False:
                from ..parallel.symmetric import SymmetricHeap
                from .tensor_parallel import TensorParallelResidency

                heap = SymmetricHeap(cpu_group=self._group, rank=rank, world_size=world,
                                     nbytes=TensorParallelResidency.required_heap_bytes(spec), device=device)
                transport = P2PTransport(heap)
            else:
                transport = CollectiveTransport(self._group, rank, world)
        super().__init__(spec, device=device, owners=bindings.owners, my_rank=rank, transport=transport,
                         heap=heap, options=bindings.execution_options,
                         host_pool_factory=bindings.allocate_host_record_storage,
                         replicated_selections=bindings.native_selections_replicated)
        self.world = world
        self.writes_replicated = bindings.native_record_writes_replicated
        self._loc_all = {}          # group -> every consumer's resolved locations (collective transports)

    def _check_agreement(self, spec, bindings):
        """Every owner must have been configured identically; disagreement is a start-up error."""
        import torch.distributed as dist

        mine = (spec.capacity_plan.device_record_capacity, spec.capacity_plan.host_record_capacity,
                spec.layer_reuse.layer_count, spec.storage_layout.bytes_per_token,
                bindings.native_record_writes_replicated, bindings.native_selections_replicated,
                bindings.stripe_shift)
        everyone = [None] * bindings.world_size
        dist.all_gather_object(everyone, mine, group=self._group)
        if any(e != mine for e in everyone):
            raise RuntimeError(f"Record owners disagree on the cache configuration: {everyone}")

    def plan(self, layer: int, access: SparseAttentionAccessPlan):
        import torch

        g = self.groups.group(layer)
        if g in self._loc or self.world == 1 or self.replicated_selections:
            return super().plan(layer, access)
        import torch.distributed as dist

        # export: every consumer's selection reaches every owner
        sel = access.selected_logical_record_ids.to(torch.int32).contiguous()
        cur = access.current_logical_record_ids
        a = self.spec.sparse_access
        padded = torch.zeros((a.maximum_padded_query_count, a.maximum_selected_record_count + 1),
                             dtype=torch.int32, device=sel.device)
        padded[:sel.shape[0], :sel.shape[1]] = sel
        if cur is not None:
            padded[:cur.numel(), -1] = cur.reshape(-1).to(torch.int32)
        everyone = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(everyone, padded, group=self._group)
        union = torch.stack(everyone)
        res = self.residency[g]
        res.pin(union)
        res.plan_step()
        self._exchange_group(g, layer)
        res.commit()
        self.transport.barrier()
        if self.transport.kind == "collective":
            # Peers' directories are not addressable: every owner resolves EVERY consumer's selection
            # for the records it owns, an element-wise max combines the owners' answers, and each
            # consumer keeps its own slice (all of it stays around for the record gather below).
            k = a.maximum_selected_record_count
            owned = self._resolve(g, layer, union[:, :, :k].contiguous(), merge=False)
            everyone_loc = self.transport.merge_locations(owned)
            self._loc_all[g] = everyone_loc
            loc = everyone_loc[self.my_rank, :sel.shape[0], :sel.shape[1]].contiguous()
        else:
            loc = self._resolve(g, layer, sel)
        self._loc[g] = loc
        self._sel[g] = sel
        return loc

    def gather_window(self, layer: int):
        """Independent selections over a collective transport: owners contribute the rows of every
        consumer's selection, a sum assembles them, each consumer keeps its own window."""
        import torch

        g = self.groups.group(layer)
        if (self.world == 1 or self.replicated_selections or self.transport.kind != "collective"
                or g not in self._loc_all):
            return super().gather_window(layer)
        everyone = self._loc_all[g]
        window = self.transport.gather_window(self, layer, everyone)
        q, k = self._sel[g].shape
        per = everyone.shape[1] * everyone.shape[2]
        mine = window[self.my_rank * per:(self.my_rank + 1) * per].view(everyone.shape[1], everyone.shape[2], -1)
        return mine[:q, :k].reshape(q * k, -1).contiguous()

    def write(self, layer, ids, values, *, owner_only=None):
        """Replicated writers: only the owner stores.  Independent writers on a symmetric
        heap store straight into the owner's pool; over collectives the records are
        all-gathered and each owner keeps its share."""
        import torch

        if self.world == 1 or self.writes_replicated:
            return super().write(layer, ids, values, owner_only=True)
        if self.transport.kind == "p2p":
            return super().write(layer, ids, values, owner_only=False)
        import torch.distributed as dist
        from ..ops import records

        plane = self.planes[0]
        rows = values if torch.is_tensor(values) and values.dtype == torch.uint8 else \
            records.ENCODERS[plane.native_encoding](*values)
        cap = self.spec.capacity_plan.maximum_write_record_count
        buf = torch.zeros((cap, rows.shape[1]), dtype=torch.uint8, device=rows.device)
        idb = torch.zeros((cap,), dtype=torch.int32, device=rows.device)
        n = rows.shape[0]
        buf[:n], idb[:n] = rows, ids.reshape(-1).to(torch.int32)
        all_rows = [torch.empty_like(buf) for _ in range(self.world)]
        all_ids = [torch.empty_like(idb) for _ in range(self.world)]
        dist.all_gather(all_rows, buf, group=self._group)
        dist.all_gather(all_ids, idb, group=self._group)
        super().write(layer, torch.cat(all_ids), torch.cat(all_rows), owner_only=True)

    def close(self):
        super().close()
        if self.heap is not None:
            self.heap.close()
            self.heap = None
