"""Rank-local engine over native page layouts: several record planes, caller-supplied record unions,
eager prefill unions, receive rows, native-page publication and storage inventories.

A serving framework that keeps its own paged KV pool ("native pages") uses this engine as the residency
layer under those pages.  On top of the common transaction of :class:`CacheEngine` (pin -> plan ->
exchange -> commit -> resolve) it offers what such an integration needs:

* ``prepare_record_residency(domain, ids)`` / ``finish_record_residency(domain)`` - make a CALLER-supplied
  list of owner-local ids resident (repeats and negative padding allowed, de-duplicated here), lease the
  residency domain until the caller's readers have retired, and refuse to replace a domain that is live;
* ``plan_prefill(layer, selection)`` - the eager prefill form: one union per selection producer and
  forward, bound-checked against the startup budget, answered with the selection rewritten as device
  rows; ``prepare_prefill_record_chunk`` / ``finish_prefill_record_chunk`` borrow one resident chunk for
  a reconstruction read;
* ``allocate_receive_rows(ids)`` - bind unpublished destinations in the host tier for records that will
  arrive from elsewhere (a prefill worker, a snapshot), returning the host rows to write;
* ``write_native_paged_records`` - publish records that already sit, encoded, in the framework's pages;
* ``device_storage_inventory`` / ``host_storage_inventory`` / ``memory_inventory`` - every allocation by
  address and size, so a launcher can reconcile the cache's footprint with its memory budget.

Reference: NativePagedResidency (ulacache/cache/local_paged_cache.py:9-761; allocate_receive_rows :244,
prepare_record_residency :479, plan_prefill :533, prepare_prefill_record_chunk :602,
write_native_paged_records :655, device_storage_inventory :685, memory_inventory :731).
"""
from __future__ import annotations

from ..storage.layout import OwnerMap
from .engine import CacheEngine


class NativePagedResidency(CacheEngine):
    def __init__(self, spec, bindings):
        super().__init__(spec, device=bindings.device, owners=OwnerMap(1, 6), my_rank=0,
                         options=bindings.execution_options,
                         host_pool_factory=bindings.allocate_host_record_storage)
        self._live_domains = {}          # residency group -> what holds it ("union", "prefill", "chunk")
        self._prefill_planned = set()    # groups whose prefill union was planned in this forward
        self._union_ws = {}

    # --------------------------------------------------------------------- views --
    @property
    def device_record_planes_by_layer(self):
        return tuple(tuple(self.layer_plane(l, p) for p in range(len(self.planes)))
                     for l in range(self.spec.layer_reuse.layer_count))

    def get_device_record_planes(self, layer: int):
        """Borrowed device views of every record plane of ``layer`` (aliased layers share storage)."""
        return self.device_record_planes_by_layer[layer]

    @property
    def device_record_banks_by_layer(self):
        """One view per layer; only meaningful for a single-plane layout."""
        if len(self.planes) > 1:
            raise ValueError("use get_device_record_planes for a cache with separate native planes")
        return tuple(self.layer_plane(l) for l in range(self.spec.layer_reuse.layer_count))

    @property
    def supports_local_native_current_publication(self) -> bool:
        """Whether a freshly produced record can be published through the directory in the same launch
        that encodes it (true on GPUs: ``kv_write`` resolves the id itself)."""
        return self.is_cuda

    # ------------------------------------------------------------------ lifetime --
    def require_idle(self, what: str):
        super().require_idle(what)
        if self._live_domains:
            raise RuntimeError(f"Finish every record reader before {what} "
                               f"(live residency domains: {sorted(self._live_domains)})")

    def begin_forward(self, context=None):
        super().begin_forward(context)
        self._prefill_planned.clear()

    def allocate_receive_rows(self, ids, *, order_free_tail: bool = True):
        """Register ``ids`` in the HOST tier without publishing payloads and return their host rows
        (int64 [n]): the receiver writes ``layer_host_plane(layer)[rows]`` and the records become
        readable with the next residency transaction.  ``order_free_tail``: first sort the top of the free
        stack, so that the rows come out ascending and mostly adjacent and a transport can write them as a few
        contiguous extents."""
        import torch

        self.require_idle("binding receive rows")
        if self._geom.host_slots <= 0:
            raise RuntimeError("receive rows live in the host tier, which this cache was built without")
        flat = ids.reshape(-1)
        for res in self.residency:
            if order_free_tail:
                res.order_host_free_tail(int(flat.numel()))
            res.register(flat, prefer_device=False)
        res = self.residency[0]
        mine, local = res._owned_locals(flat.to(torch.int32).to(res.directory.device))
        entry = res.directory[local.long()]
        if bool((entry > -2).any()):
            raise MemoryError("the host tier could not take every receive row")
        return (-entry.long() - 2)

    # ------------------------------------------------------- caller-supplied union --
    def _bounded_union(self, ids):
        import torch

        flat = ids.reshape(-1)
        cap = self.spec.capacity_plan
        if flat.numel() > cap.maximum_residency_input_record_count:
            raise ValueError("record union input exceeds its startup bound "
                             f"({flat.numel()} > {cap.maximum_residency_input_record_count})")
        if flat.is_cuda:
            from ..ops import prefill as P

            space = (cap.logical_record_capacity + 1) * self.owners.ranks + self.owners.allocation_page
            f32 = flat.to(torch.int32)
            f32 = torch.where(f32 > 0, f32, torch.full_like(f32, -1))
            uni, count, _ = P.selection_union(f32, space, capacity=min(f32.numel(), space), workspace=self._union_ws)
            uni = uni[: int(count)]
        else:
            uni = torch.unique(flat[flat > 0].to(torch.int32), sorted=True)
        if uni.numel() > cap.device_record_capacity:
            raise ValueError(f"complete record union ({uni.numel()}) exceeds the device tier "
                             f"({cap.device_record_capacity} records)")
        return uni

    def _transact(self, g: int, union_ids):
        """pin -> plan -> exchange -> commit of ``union_ids`` on residency group ``g``."""
        if self._geom.host_slots > 0 and union_ids.numel():
            res = self.residency[g]
            if not self._forward_open:
                res.begin_step()
            res.pin(union_ids.reshape(1, -1))
            res.plan_step()
            self._exchange_group(g, self.groups.anchors[g])
            res.commit()

    def prepare_record_residency(self, domain: int, owner_local_record_ids):
        """Lease residency ``domain`` (a residency group) for a caller-supplied record list.  Returns the
        de-duplicated ids (ascending) and their device rows.  The domain stays leased until
        :meth:`finish_record_residency`; replacing a live domain is refused."""
        if not 0 <= domain < self.groups.group_count:
            raise IndexError("residency domain outside the cache")
        if domain in self._live_domains:
            raise RuntimeError("Finish the current record union before replacing its residency")
        uni = self._bounded_union(owner_local_record_ids)
        self._transact(domain, uni)
        self._live_domains[domain] = "union"
        rows = self._device_rows(domain, uni)
        return uni, rows

    def finish_record_residency(self, domain: int):
        if self._live_domains.pop(domain, None) is None:
            raise RuntimeError("this residency domain holds no record union")

    def _device_rows(self, g: int, ids):
        """Device row of every id (-1 for padding or non-resident), shaped like ``ids``."""
        import torch

        layer = self.groups.anchors[g]
        loc = self._resolve(g, layer, ids.to(torch.int32).reshape(1, -1) if ids.ndim == 1 else ids.to(torch.int32))
        rows = torch.where(loc >= 0, loc & 0x0FFFFFFF, torch.full_like(loc, -1))
        return rows.reshape(ids.shape)

    # ------------------------------------------------------------------- prefill --
    def plan_prefill(self, layer: int, selected_logical_records):
        """Eager prefill: make the UNION of the selection resident (once per selection producer and forward;
        bytes written before planning are preserved) and return the selection as device rows."""
        import torch

        if self.is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the prefill union requires eager execution")
        g = self.groups.group(layer)
        if g not in self._prefill_planned:
            if g in self._live_domains:
                raise RuntimeError("the previous selection on this residency domain still has readers")
            self._transact(g, self._bounded_union(selected_logical_records))
            self._prefill_planned.add(g)
            self._live_domains[g] = "prefill"
        return self._device_rows(g, selected_logical_records)

    def prepare_prefill_record_chunk(self, layer: int, logical_record_ids):
        """Borrow one resident chunk of records until its reconstruction read has finished."""
        g = self.groups.group(layer)
        if g in self._live_domains:
            raise RuntimeError("finish the current domain reader before replacing its prefill records")
        self._transact(g, self._bounded_union(logical_record_ids))
        self._live_domains[g] = "chunk"
        return self._device_rows(g, logical_record_ids)

    def finish_prefill_record_chunk(self, layer: int):
        g = self.groups.group(layer)
        if self._live_domains.get(g) != "chunk":
            raise RuntimeError("no prefill record chunk is borrowed on this layer's domain")
        del self._live_domains[g]

    def after_attention(self, layer: int):
        super().after_attention(layer)
        g = self.groups.group(layer)
        last = self.groups.layers_of(g)[-1]
        if layer == last and self._live_domains.get(g) == "prefill":
            del self._live_domains[g]

    # --------------------------------------------------------------------- write --
    def write_native_paged_records(self, layer: int, ids, pages, source_indices, *,
                                   local_device_after_commit: bool = False):
        """Publish records that already sit, encoded, in native pages: ``pages`` is a uint8 tensor
        ``[n_pages * 64, record_bytes]`` (or [n_pages, 64, record_bytes]) and ``source_indices`` picks rows.
        ``local_device_after_commit``: the caller asserts that a committed transaction has just made every
        id device-resident here; a record that is not is an error instead of a host-tier write."""
        import torch

        rows = pages.reshape(-1, pages.shape[-1])[source_indices.reshape(-1).long()]
        if local_device_after_commit:
            g = self.groups.group(layer)
            res = self.residency[g]
            _, local = res._owned_locals(ids.reshape(-1).to(torch.int32).to(res.directory.device))
            if bool((res.directory[local.long()] < 0).any()):
                raise RuntimeError("a record promised to be device-resident after commit is not")
        self.write(layer, ids, rows)

    def offload_prefill(self, ids):
        """Move finished prefill records to the host tier (single-plane layouts)."""
        if len(self.planes) > 1:
            raise NotImplementedError("paged records with separate planes keep their final prefill residency")
        from .local_cache import UnifiedLocalResidency

        return UnifiedLocalResidency.offload_prefill(self, ids)

    # ----------------------------------------------------------------- inventory --
    def _metadata_tensors(self):
        out = []
        for res in self.residency:
            out.extend(getattr(res, k) for k in res.STATE)
        if self.status is not None:
            out.extend((self.status, self._not_resident))
        for v in self._union_ws.values():
            if hasattr(v, "untyped_storage"):
                out.append(v)
        return out

    def device_storage_inventory(self) -> dict:
        """{storage address: bytes} of every device allocation the cache holds (payload and metadata);
        aliases of one storage count once."""
        inv = {}
        tensors = [st.gpu for st in self.storages] + self._metadata_tensors()
        for t in tensors:
            if t is not None and t.numel() and t.device.type == self.device.type:
                s = t.untyped_storage()
                inv[s.data_ptr()] = max(inv.get(s.data_ptr(), 0), s.nbytes())
        return inv

    def host_storage_inventory(self) -> dict:
        inv = {}
        for st in self.storages:
            h = st.host
            if h is not None and h.numel():
                s = h.untyped_storage()
                inv[s.data_ptr()] = max(inv.get(s.data_ptr(), 0), s.nbytes())
        return inv

    def memory_inventory(self) -> dict:
        inv = super().memory_inventory()
        dev = self.device_storage_inventory()
        inv["gpu_bytes"] = sum(dev.values()) if self.is_cuda else 0
        inv["gpu_kv_bytes"] = inv["device_key_value_bytes"] if self.is_cuda else 0
        inv["gpu_metadata_bytes"] = max(0, inv["gpu_bytes"] - inv["gpu_kv_bytes"])
        inv["host_bytes"] = sum(self.host_storage_inventory().values())
        inv["residency_directory_count"] = len(self.residency)
        inv["selection_producer_count"] = self.groups.group_count
        inv["record_planes"] = len(self.planes)
        inv["live_residency_domains"] = sorted(self._live_domains)
        return inv
