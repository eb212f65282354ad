"""The residency engine shared by every execution mode.

One engine owns, for one rank:

* the KV record planes (HBM + pinned host) of the layers that own storage,
* one :mod:`residency` group per shared-selection layer group,
* the per-forward transaction ``begin_forward -> plan(layer) -> write ->
  attention_rows(layer) -> after_attention(layer) -> finish_forward``.

Modes differ only in the owner map and in how peers are reached:

===================  =========================  =====================================
mode                 owner map                  peers
===================  =========================  =====================================
local (DPA)          1 owner                    none
paged                1 owner, several planes    none
position (CP)        1 owner per rank, IDs are  none (partial O/LSE merged later)
                     localised first
tensor parallel      N owners, page-striped     replicated selections; every owner
                                                promotes its share, consumers read
                                                peers' directories and pools
record owner         N owners                   independent selections exported to
                                                the owners first
===================  =========================  =====================================

Peer data is reached through a *transport*: ``P2PTransport`` (peer pointers from
the symmetric heap, the product path) or ``CollectiveTransport``
(``torch.distributed`` all-reduce / all-gather over NCCL or gloo: the baseline
and the CPU test path).

Reference: engine protocol of ulacache/cache/local_cache.py:208-649 (DPA),
ulacache/cache/tp_cache.py:389-519 + ulacache/cache/prefetch.py:4-219 (TP),
ulacache/cache/owner_cache.py:323-457 (owners).
"""
from __future__ import annotations

from typing import Optional

from ..cache_config import CacheExecutionOptions
from ..storage.buffers import RecordPlaneStorage, default_host_pool_factory
from ..storage.layout import KERNEL_FORMAT_CODE, OwnerMap, PAGE_TOKENS
from .access import ResidentAttentionInputs, SparseAttentionAccessPlan
from .residency import CNT_PLAN, CNT_UNSERVED, ResidencyGeometry, make_residency
from .specification import UnifiedCacheSpecification


class CollectiveTransport:
    """Peers reached with ``torch.distributed`` collectives (NCCL on GPU, gloo on CPU)."""

    kind = "collective"

    def __init__(self, group, rank, world):
        self.group, self.rank, self.world = group, rank, world

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier(group=self.group)

    def merge_locations(self, loc):
        """Each rank resolved only what it owns (-1 elsewhere): element-wise max merges."""
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(loc, op=dist.ReduceOp.MAX, group=self.group)
        return loc

    def gather_window(self, engine, layer, loc):
        """Dense ``[n, record_bytes]`` window of the records named by ``loc``: every owner
        contributes its rows, zero elsewhere, and a sum all-reduce assembles them."""
        import torch

        flat = loc.reshape(-1)
        plane = engine.layer_plane(layer)
        rank_of = (flat >> 28) & 0x7
        mine = (flat >= 0) & (rank_of == self.rank)
        window = torch.zeros((flat.numel(), plane.shape[-1]), dtype=torch.uint8, device=plane.device)
        window[mine] = plane[(flat[mine] & 0x0FFFFFFF).long()]
        if self.world > 1:
            import torch.distributed as dist

            w32 = window.view(torch.int32)
            dist.all_reduce(w32, op=dist.ReduceOp.SUM, group=self.group)
        return window


class P2PTransport:
    """Peers reached through pointers into their slabs (CUDA IPC over NVLink)."""

    kind = "p2p"

    def __init__(self, heap):
        self.heap, self.rank, self.world = heap, heap.rank, heap.world

    def barrier(self):
        self.heap.device_barrier()

    def merge_locations(self, loc):
        return loc      # the resolve kernel already read the peers' directories


class CacheEngine:
    def __init__(self, spec: UnifiedCacheSpecification, *, device, owners: Optional[OwnerMap] = None,
                 my_rank: int = 0, transport=None, heap=None,
                 options: Optional[CacheExecutionOptions] = None,
                 host_pool_factory=default_host_pool_factory, replicated_selections: bool = True):
        import torch

        self.spec = spec
        self.device = torch.device(device)
        self.owners = owners or OwnerMap(1, 6)
        self.my_rank = my_rank
        self.transport = transport
        self.heap = heap
        self.options = options or CacheExecutionOptions()
        self.replicated_selections = replicated_selections
        self.is_cuda = self.device.type == "cuda"
        cap = spec.capacity_plan
        reuse = spec.layer_reuse
        self.groups = reuse.residency_groups()
        # storage index of each layer (layers may alias KV storage)
        storage_ids = sorted(set(reuse.key_value_storage_owners))
        self._storage_of_layer = tuple(storage_ids.index(o) for o in reuse.key_value_storage_owners)
        self.planes = spec.storage_layout.record_planes
        self.storages = []
        for plane in self.planes:
            if heap is not None and self.is_cuda:
                st = _HeapPlaneStorage(plane, heap=heap, layers=len(storage_ids),
                                       hbm_slots=cap.device_record_capacity,
                                       host_slots=cap.host_record_capacity,
                                       host_pool_factory=host_pool_factory)
            else:
                st = RecordPlaneStorage(plane, layers=len(storage_ids), hbm_slots=cap.device_record_capacity,
                                        host_slots=cap.host_record_capacity, device=self.device,
                                        host_pool_factory=host_pool_factory)
            self.storages.append(st)
        self.gpu = self.storages[0].gpu
        logical = (cap.logical_record_capacity + 1) * self.owners.ranks + self.owners.allocation_page
        geom = ResidencyGeometry(dir_len=self.owners.local_count(logical), hbm_slots=cap.device_record_capacity,
                                 host_slots=cap.host_record_capacity, plan_capacity=spec.plan_capacity)
        self.residency = []
        for g in range(self.groups.group_count):
            res = make_residency(geom, self.owners, my_rank, self.device)
            if heap is not None and self.is_cuda:
                shared = heap.alloc(f"directory.{g}.{id(self)}", (geom.dir_len,), torch.int32)
                shared.copy_(res.directory)
                res.directory = shared
                if hasattr(res, "native_state"):
                    res.native_state.directory = shared.data_ptr()
            self.residency.append(res)
        self._geom = geom
        self._loc = {}             # group -> int32 [Q, K] resolved locations of this forward
        self._sel = {}
        self._live_layers = set()
        self._forward_open = False
        self._wrote_layers = set()
        self._side_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self._layer_events = {}
        self._views = {}
        self.status = None
        if self.is_cuda:
            from ..ops import _native as N

            self.status = N.new_status(self.device)
            self._not_resident = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.closed = False

    # ------------------------------------------------------------------ helpers --
    def layer_plane(self, layer: int, plane: int = 0):
        return self.storages[plane].gpu[self._storage_of_layer[layer]]

    def layer_host_plane(self, layer: int, plane: int = 0):
        h = self.storages[plane].host
        return None if h is None else h[self._storage_of_layer[layer]]

    def _pool_view(self, layer: int, plane: int = 0):
        key = (layer, plane)
        v = self._views.get(key)
        if v is not None:
            return v
        from ..ops import records

        st = self.storages[plane]
        g = self.groups.group(layer)
        res = self.residency[g]
        local_plane = self.layer_plane(layer, plane)
        if self.heap is not None and self.owners.ranks > 1 and self.transport is not None and self.transport.kind == "p2p":
            hbm = self.heap.peer_ptrs(local_plane)
            dirs = self.heap.peer_ptrs(res.directory)
        else:
            hbm = [local_plane.data_ptr()] * self.owners.ranks
            dirs = [res.directory.data_ptr()] * self.owners.ranks
        hostp = self.layer_host_plane(layer, plane)
        v = records.make_pool_view(hbm_ptrs=hbm, dir_ptrs=dirs, host_ptr=0 if hostp is None else hostp.data_ptr(),
                                   dir_len=self._geom.dir_len, hbm_slots=self._geom.hbm_slots,
                                   host_slots=self._geom.host_slots, rec_bytes=st.plane.bytes_per_record,
                                   owners=self.owners, my_rank=self.my_rank)
        self._views[key] = v
        return v

    # ------------------------------------------------------- lifetime of records --
    def allocate_unbound(self, ids, prefer_gpu: bool = True):
        for res in self.residency:
            res.register(ids, prefer_device=prefer_gpu)

    def release(self, ids):
        self.require_idle("releasing records")
        for res in self.residency:
            res.release(ids)

    def clear(self):
        self.require_idle("clearing the cache")
        for res in self.residency:
            res.reset()
        self._loc.clear()

    def require_idle(self, what: str):
        if self._live_layers:
            raise RuntimeError(f"Finish every attention reader before {what}")

    # ------------------------------------------------------------------ forward --
    def begin_forward(self, context=None):
        self.require_idle("beginning another forward")
        if self._geom.host_slots > 0:
            for res in self.residency:
                res.begin_step()
        self._wrote_layers = set()
        self._loc.clear()
        self._sel.clear()
        self._layer_events.clear()
        self._forward_open = True

    def plan(self, layer: int, access: SparseAttentionAccessPlan):
        """Make every selected record of ``layer``'s group resident in HBM (on its
        owner) and resolve the selection to physical locations.  Runs the whole
        transaction for the group's anchor; follower layers reuse the result."""
        import torch

        g = self.groups.group(layer)
        if g in self._loc:
            return self._loc[g]
        res = self.residency[g]
        sel = access.selected_logical_record_ids
        cur = access.current_logical_record_ids
        if self._geom.host_slots > 0:
            res.pin(sel)
            if cur is not None:
                res.pin(cur)
            res.plan_step()
            self._exchange_group(g, layer)
            res.commit()
            if self.transport is not None and self.owners.ranks > 1:
                self.transport.barrier()       # every owner has committed before anyone resolves
        # without a host tier nothing can move: directories change only when records are
        # registered or released, outside forwards, so resolving needs no transaction
        loc = self._resolve(g, layer, sel)
        self._loc[g] = loc
        self._sel[g] = sel
        return loc

    def _exchange_group(self, g: int, anchor_layer: int):
        res = self.residency[g]
        if self._geom.host_slots == 0:
            return
        layers = self.groups.layers_of(g)
        storage_layers = sorted({self._storage_of_layer[l] for l in layers})
        if not self.is_cuda:
            from ..ops.exchange import exchange_reference

            for st in self.storages:
                exchange_reference(res.plan_items(), st.gpu, st.host, storage_layers)
            return
        import torch
        from ..ops import exchange as X

        blocks, threads = self.options.exchange_launch_dimensions
        lo, hi = storage_layers[0], storage_layers[-1] + 1
        async_followers = self.options.copy_follower_records_asynchronously and hi - lo > 1
        for st in self.storages:
            rb = st.plane.bytes_per_record
            if not async_followers:
                X.exchange(res.native_state, X.make_plane_set(st.gpu, st.host, rb, lo, hi - lo), blocks, threads)
                continue
            a = self._storage_of_layer[anchor_layer]
            X.exchange(res.native_state, X.make_plane_set(st.gpu, st.host, rb, a, 1), blocks, threads)
        if async_followers:
            # followers move on the side stream while the anchor layer computes
            main = torch.cuda.current_stream()
            ready = torch.cuda.Event()
            ready.record(main)
            self._side_stream.wait_event(ready)
            fb, ft = self.options.follower_exchange_launch_dimensions or (blocks, threads)
            with torch.cuda.stream(self._side_stream):
                a = self._storage_of_layer[anchor_layer]
                per_layer = self.options.follower_copy_mode == "layer"
                followers = [l for l in range(lo, hi) if l != a]
                for st in self.storages:
                    rb = st.plane.bytes_per_record
                    if per_layer:
                        for l in followers:
                            X.exchange(res.native_state, X.make_plane_set(st.gpu, st.host, rb, l, 1), fb, ft)
                    else:
                        runs = _contiguous_runs(followers)
                        for s, n in runs:
                            X.exchange(res.native_state, X.make_plane_set(st.gpu, st.host, rb, s, n), fb, ft)
                done = torch.cuda.Event()
                done.record(self._side_stream)
            for l in self.groups.layers_of(g):
                if self._storage_of_layer[l] != a:
                    self._layer_events[l] = done

    def _resolve(self, g: int, layer: int, sel, *, merge: bool = True):
        """Physical locations of ``sel``.  ``merge=False`` (collective transports): only what this
        rank owns, -1 elsewhere; the caller combines the owners' answers itself."""
        import torch

        res = self.residency[g]
        if self.is_cuda:
            from ..ops import exchange as X

            loc = torch.empty(sel.shape, dtype=torch.int32, device=self.device)
            X.resolve(self._pool_view(layer), sel.contiguous(), loc, not_resident=self._not_resident,
                      status=self.status)
            if self.transport is not None and self.transport.kind == "collective" and self.owners.ranks > 1:
                # peers' directories are not addressable: keep only what this rank owns, then merge
                owner = (sel >> self.owners.stripe_shift) % self.owners.ranks
                loc = torch.where((sel > 0) & (owner == self.my_rank), loc, torch.full_like(loc, -1))
                if merge:
                    loc = self.transport.merge_locations(loc)
            return loc
        ids = sel.to(torch.int32)
        mine, local = res._owned_locals(ids.reshape(-1))
        loc = torch.full((ids.numel(),), -1, dtype=torch.int32, device=self.device)
        e = res.directory[local[mine].long()]
        ok = e >= 0
        vals = torch.where(ok, (self.my_rank << 28) | e, torch.full_like(e, -1))
        loc[mine] = vals
        loc = loc.view(sel.shape)
        if merge and self.transport is not None and self.owners.ranks > 1:
            loc = self.transport.merge_locations(loc)
        return loc

    def before_layer_consume(self, layer: int):
        """Make the current stream wait for the layer's asynchronous exchange, if any."""
        ev = self._layer_events.get(layer)
        if ev is not None:
            import torch

            torch.cuda.current_stream().wait_event(ev)

    def attention_rows(self, layer: int) -> ResidentAttentionInputs:
        g = self.groups.group(layer)
        if g not in self._loc:
            raise RuntimeError("plan() the layer's selection before asking for attention rows")
        self.before_layer_consume(layer)
        if (layer in getattr(self, "_wrote_layers", ()) and self.transport is not None
                and self.transport.kind == "p2p" and self.owners.ranks > 1 and getattr(self, "remote_readers", True)):
            # peers read this step's freshly written records straight from the owner's pool:
            # every owner's write must have landed before any rank starts its attention kernel
            self.transport.barrier()
            self._wrote_layers.discard(layer)
        self._live_layers.add(layer)
        planes = tuple(self.layer_plane(layer, p) for p in range(len(self.planes)))
        peer = ()
        view = None
        if self.is_cuda:
            view = self._pool_view(layer)
            peer = tuple(view.hbm[r] or 0 for r in range(self.owners.ranks))
        return ResidentAttentionInputs(record_planes=planes, device_record_indices=self._loc[g],
                                       records_per_page=PAGE_TOKENS,
                                       record_layout="segment_major" if self.planes[0].segment_major else "record_major",
                                       peer_planes=peer, pool_view=view)

    def gather_window(self, layer: int):
        """Dense copy of the layer's selected records (decoded by the caller); used by
        the baseline path and the CPU reference."""
        import torch

        g = self.groups.group(layer)
        loc = self._loc[g]
        if self.transport is not None and self.transport.kind == "collective" and self.owners.ranks > 1:
            return self.transport.gather_window(self, layer, loc)
        plane = self.layer_plane(layer)
        flat = loc.reshape(-1)
        if self.is_cuda:
            from ..ops import exchange as X

            out = torch.empty((flat.numel(), plane.shape[-1]), dtype=torch.uint8, device=self.device)
            X.gather_locations(self._pool_view(layer), flat.contiguous(), out, status=self.status)
            return out
        out = torch.zeros((flat.numel(), plane.shape[-1]), dtype=torch.uint8, device=self.device)
        ok = flat >= 0
        out[ok] = plane[(flat[ok] & 0x0FFFFFFF).long()]
        return out

    def read_records(self, layer: int, ids):
        """Read-only: the stored bytes of logical ``ids`` for ``layer`` as this rank can reach them
        (its HBM or host tier; on GPUs also peers' HBM) -> (uint8 [n, record bytes], bool [n] found);
        on GPUs a third value, the device count of ids that could not be read.
        Changes no residency state: used by prefill readers and snapshot writers."""
        import torch

        ids = ids.reshape(-1).to(torch.int32)
        plane = self.layer_plane(layer)
        out = torch.zeros((ids.numel(), plane.shape[-1]), dtype=torch.uint8, device=self.device)
        if self.is_cuda:
            from ..ops import prefill as P

            missing = torch.zeros(1, dtype=torch.int32, device=self.device)
            P.gather_by_directory(self._pool_view(layer), ids.contiguous(), out, missing=missing, status=self.status)
            return out, (ids >= 0), missing
        res = self.residency[self.groups.group(layer)]
        mine, local = res._owned_locals(ids)
        found = torch.zeros(ids.numel(), dtype=torch.bool, device=self.device)
        e = res.directory[local[mine].long()]
        on_dev, on_host = e >= 0, e <= -2
        rows = mine.nonzero().flatten()
        out[rows[on_dev]] = plane[e[on_dev].long()]
        hostp = self.layer_host_plane(layer)
        if hostp is not None and bool(on_host.any()):
            out[rows[on_host]] = hostp[(-e[on_host] - 2).long()].to(self.device)
            found[rows[on_host]] = True
        found[rows[on_dev]] = True
        return out, found

    def after_attention(self, layer: int):
        self._live_layers.discard(layer)

    def finish_forward(self):
        self.require_idle("finishing the forward")
        if self.is_cuda and self._layer_events:
            import torch

            for ev in set(self._layer_events.values()):
                torch.cuda.current_stream().wait_event(ev)
        self._forward_open = False

    def abort_forward(self):
        """Drop the forward's reader state after an error: join the side stream, forget views."""
        if self.is_cuda:
            import torch

            self._side_stream.synchronize()
            torch.cuda.current_stream().synchronize()
        self._live_layers.clear()
        self._loc.clear()
        self._layer_events.clear()
        self._forward_open = False

    # -------------------------------------------------------------------- write --
    def write(self, layer: int, ids, values, *, owner_only: bool = True):
        """Encode and publish the KV of ``ids`` for ``layer``.  ``values`` = (latent, rope)
        float tensors, or a uint8 ``[n, record_bytes]`` tensor of already-encoded records."""
        import torch

        self.before_layer_consume(layer)
        if self._forward_open:
            getattr(self, "_wrote_layers", set()).add(layer)
        plane = self.planes[0]
        encoded = torch.is_tensor(values) and values.dtype == torch.uint8
        if self.is_cuda:
            from ..ops import records

            view = self._pool_view(layer)
            ids32 = ids.reshape(-1).to(torch.int32).contiguous()
            if encoded:
                records.kv_write_encoded(view, values.contiguous(), ids32, owner_only=owner_only, status=self.status)
            else:
                latent, rope = values
                records.kv_write(view, KERNEL_FORMAT_CODE[plane.native_encoding],
                                 latent.to(torch.bfloat16).contiguous(), rope.to(torch.bfloat16).contiguous(),
                                 ids32, owner_only=owner_only, status=self.status)
            return
        from ..ops import records

        rows = values if encoded else records.ENCODERS[plane.native_encoding](*values)
        g = self.groups.group(layer)
        res = self.residency[g]
        ids32 = ids.reshape(-1).to(torch.int32)
        mine, local = res._owned_locals(ids32)
        e = res.directory[local[mine].long()]
        src = rows[mine]
        gp, hp = self.layer_plane(layer), self.layer_host_plane(layer)
        on_dev = e >= 0
        gp[e[on_dev].long()] = src[on_dev]
        on_host = e <= -2
        if on_host.any():
            hp[(-e[on_host] - 2).long()] = src[on_host].cpu()
        if (e == -1).any():
            raise RuntimeError("writing to an unallocated record")

    # ---------------------------------------------------------------- inventory --
    def memory_inventory(self) -> dict:
        dev = sum(st.device_bytes() for st in self.storages)
        host = sum(st.host_bytes() for st in self.storages)
        meta = sum(r.metadata_bytes() for r in self.residency)
        cap = self.spec.capacity_plan
        return {
            "device_key_value_bytes": dev,
            "host_key_value_bytes": host,
            "metadata_bytes": meta,
            "device_record_capacity": cap.device_record_capacity,
            "host_record_capacity": cap.host_record_capacity,
            "logical_record_capacity": cap.logical_record_capacity * self.owners.ranks,
            "residency_groups": self.groups.group_count,
            "owners": self.owners.ranks,
            "rank": self.my_rank,
        }

    storage_inventory = memory_inventory

    def counters(self) -> dict:
        out = {}
        for g, r in enumerate(self.residency):
            for k, v in r.stats().items():
                out[k] = out.get(k, 0) + v if k not in ("epoch",) else v
        return out

    def check(self, what="cache step"):
        """Read back device status words (synchronises); raises on any kernel-reported error, and, in the
        canary build of the storage, on an overwritten guard record."""
        for st in self.storages:
            check = getattr(st, "check_canaries", None)
            if check is not None:
                check()
        if not self.is_cuda:
            return
        from ..ops import _native as N

        N.raise_on_status(self.status, what)
        for r in self.residency:
            r.check_status(what)

    def close(self):
        if self.closed:
            return
        if self.is_cuda:
            import torch

            self._side_stream.synchronize()
            torch.cuda.synchronize(self.device)
        if self.transport is not None and self.owners.ranks > 1 and self.transport.kind == "collective":
            self.transport.barrier()
        for st in self.storages:
            st.close()
        self.closed = True


def _contiguous_runs(values):
    runs, start, prev = [], None, None
    for v in values:
        if start is None:
            start = prev = v
        elif v == prev + 1:
            prev = v
        else:
            runs.append((start, prev - start + 1))
            start = prev = v
    if start is not None:
        runs.append((start, prev - start + 1))
    return runs


class _HeapPlaneStorage(RecordPlaneStorage):
    """Record planes carved out of the symmetric heap so that peers can address them."""

    def __init__(self, plane, *, heap, layers, hbm_slots, host_slots, host_pool_factory):
        import torch

        self.plane = plane
        from ..storage.buffers import PlaneGeometry

        self.geometry = PlaneGeometry(layers, hbm_slots, host_slots, plane.bytes_per_record)
        self.device = heap.device
        self.gpu = heap.alloc(f"plane.{plane.name}.{id(self)}", (layers, hbm_slots, plane.bytes_per_record), torch.uint8)
        self.guard, self._device_block = 0, self.gpu      # peers address these planes: no guard records in the heap
        self.host_pool = None
        if host_slots > 0:
            self.host_pool = host_pool_factory(layers=layers, slots=host_slots, row_bytes=plane.bytes_per_record,
                                               device=self.device)
