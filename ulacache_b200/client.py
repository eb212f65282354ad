"""Public cache handle: ``init`` / ``alloc`` / ``write`` / ``access`` / ``free`` plus
the forward lifecycle used by attention layers.

    cache = ulacache_b200.init(spec, bindings)
    ids = cache.alloc(n)                       # logical IDs, registered in both tiers' directory
    cache.begin_model_forward(ctx)
    cache.prepare_sparse_attention(layer, plan)  # promote + resolve (once per selection group)
    cache.write(ids, layer, (latent, rope))    # publish this step's KV
    view = cache.get_resident_attention_inputs(layer)
    ... attention kernel reads view.record_planes / view.device_record_indices ...
    cache.finish_layer_attention(layer)
    cache.finish_model_forward()
    cache.free(ids)

Reference: ulacache/client.py (init :19, alloc :82, write :93, access :163,
free :177, begin_model_forward :202, prepare_sparse_attention :270,
get_resident_attention_inputs :276, finish_layer_attention :359,
finish_model_forward :366, inventories :385-407).
"""
from __future__ import annotations

from .cache.access import ForwardExecutionContext, ResidentAttentionInputs, SparseAttentionAccessPlan
from .cache.specification import UnifiedCacheSpecification

__all__ = ["init", "UlaCache", "UnifiedMemoryCache", "ResidentView"]
ResidentView = ResidentAttentionInputs


def init(spec: UnifiedCacheSpecification, bindings):
    """Bind a specification and the framework's resources to one execution engine."""
    return UlaCache(spec, bindings)


class UnifiedMemoryCache:
    def __init__(self, cache_specification: UnifiedCacheSpecification, cache_bindings):
        from .cache.create import create_execution_engine
        from .cache.runtime import AccessEngine, PagedLogicalAllocator, SlotManager

        self.cache_specification = cache_specification
        self.cache_bindings = cache_bindings
        self._engine = create_execution_engine(cache_specification, cache_bindings)
        self._access = AccessEngine(cache_specification, self._engine)
        allocator = getattr(cache_bindings, "logical_slot_allocator", None)
        if allocator is None:
            owners = getattr(self._engine, "owners", None)
            ranks = owners.ranks if owners is not None else 1
            page = owners.allocation_page if owners is not None else 64
            cap = cache_specification.capacity_plan.usable_logical_record_capacity * ranks
            allocator = PagedLogicalAllocator(cap // page * page, page, device=self._engine.device)
        self._slots = SlotManager(self._engine, allocator, self._access)

    # ------------------------------------------------------------- five verbs --
    def _live(self):
        if self._engine is None:
            raise RuntimeError("The cache is closed")
        return self._engine

    def alloc(self, n: int):
        """Allocate ``n`` logical IDs and give each a slot (HBM first, then host).  An
        admission-time operation: call it outside forwards and graph capture."""
        self._live()
        return self._slots.alloc(n)

    def write(self, ids, layer: int, values, *, source_indices=None):
        """Publish KV for already allocated IDs on the current stream.

        ``values`` is ``(latent, rope)`` float tensors (the writer quantises), a uint8
        tensor of encoded records, native pages plus ``source_indices``, or a
        :class:`~ulacache_b200.transfer.file_io.FileRecordSource` (blocking restore
        outside forwards)."""
        engine = self._live()
        layers = self.cache_specification.layer_reuse.layer_count
        if type(layer) is not int or not 0 <= layer < layers:
            raise ValueError("Layer outside the configured cache")
        if ids.dim() != 1:
            raise ValueError("Write IDs must be a one-dimensional tensor")
        from .transfer.file_io import FileRecordSource

        if isinstance(values, FileRecordSource):
            if source_indices is not None:
                raise ValueError("A file source already names its complete record range")
            if ids.numel() != values.record_count:
                raise ValueError("Supply one logical ID per record of the file source")
            plane = self.cache_specification.storage_layout.record_planes[0]
            if values.native_encoding != plane.native_encoding or values.row_bytes != plane.bytes_per_record:
                raise ValueError("The file source does not match the cache's record encoding")
            self._access.require_idle("restoring file records")
            from .transfer.file_io import restore_file_records

            return restore_file_records(engine, layer, ids, values)
        if ids.numel() > self.cache_specification.capacity_plan.maximum_write_record_count:
            raise ValueError("Write exceeds the configured maximum write record count")
        if source_indices is not None:
            if source_indices.dim() != 1 or source_indices.numel() != ids.numel():
                raise ValueError("Supply one source index per logical ID")
            rows = values.reshape(-1, values.shape[-1])[source_indices.long()]
            return engine.write(layer, ids, rows)
        return engine.write(layer, ids, values)

    def access(self, ids, layer: int) -> ResidentAttentionInputs:
        """Make the records named by ``ids`` (int32 [queries, width]) resident and return
        the view attention reads.  Reuses the plan when the same selection was prepared."""
        self._live()
        return self._access.access(ids, layer)

    def free(self, ids):
        """Release storage of retired records and return their IDs to the allocator."""
        self._live()
        self._slots.free(ids)

    # ------------------------------------------------- registration without IDs --
    def register_logical_records(self, ids, *, prefer_device=True):
        self._slots.register(ids, prefer_device=prefer_device)

    def release_logical_records(self, ids):
        self._slots.release(ids)

    def clear_registered_records(self):
        self._slots.clear()

    # --------------------------------------------------------- forward lifecycle --
    def begin_model_forward(self, context: ForwardExecutionContext = None):
        self._live()
        self._access.begin_forward(context)

    def prepare_sparse_attention(self, layer: int, plan: SparseAttentionAccessPlan):
        self._live()
        return self._access.prepare_selection(layer, plan)

    def get_resident_attention_inputs(self, layer: int) -> ResidentAttentionInputs:
        self._live()
        return self._access.attention_inputs(layer)

    def declare_local_readers_only(self):
        """Attention on every rank reads only the records that rank owns (owner-side attention), so
        a step's freshly written records need not be visible to peers before attention starts: the
        post-write barrier of the peer-to-peer transport is skipped."""
        self._live().remote_readers = False

    # ------------------------------------------- optional engine capabilities --
    # A serving adapter calls these on every backend; an engine that has the capability runs it, one that does
    # not either ignores the hint (the ``prepare_*`` calls that only move work earlier) or refuses clearly.
    def _capability(self, name: str, why: str):
        fn = getattr(self._live(), name, None)
        if fn is None:
            raise NotImplementedError(f"{type(self._engine).__name__} has no {name}: {why}")
        return fn

    def register_receive_records(self, ids):
        """Give incoming records canonical destinations before their addresses are published to a sender."""
        return self._capability("allocate_receive_rows", "receives go through the staging window on this backend")(ids)

    def prepare_forward_current_records(self, current_ids) -> bool:
        """Hint: all layers of this forward write the same current records.  True when the engine bound them once."""
        fn = getattr(self._live(), "prepare_forward_current_records", None)
        return bool(fn(current_ids)) if fn is not None else False

    def prepare_next_residency_epochs(self):
        """Hint: retire expiring recency buckets before the forward instead of inside each layer's transaction."""
        fn = getattr(self._live(), "prepare_next_residency_epochs", None)
        if fn is not None:
            fn()

    def prepare_layer_execution(self, layer: int):
        """Wait for whatever was prefetched for ``layer`` (a no-op without a prefetcher)."""
        fn = getattr(self._live(), "before_layer_prepare", None)
        if fn is not None:
            fn(layer)

    def write_native_record_segments(self, layer: int, ids, record_segments):
        """Publish records given as their native byte segments (plane order, then segment order, scales
        included): uint8 tensors ``[n, segment bytes]`` that concatenate to whole records."""
        import torch

        parts = [seg.reshape(seg.shape[0], -1).view(torch.uint8) for seg in record_segments]
        want = self.cache_specification.storage_layout.bytes_per_token
        if sum(p.shape[1] for p in parts) != want:
            raise ValueError(f"the segments add up to {sum(p.shape[1] for p in parts)} bytes per record, not {want}")
        return self.write(ids, layer, parts[0] if len(parts) == 1 else torch.cat(parts, dim=1))

    @property
    def supports_local_native_current_publication(self) -> bool:
        return bool(getattr(self._live(), "supports_local_native_current_publication", False))

    def write_native_paged_records(self, layer: int, ids, source_record_pages, source_record_indices, *,
                                   local_device_after_commit: bool = False):
        """Publish records that sit encoded in native pages; see ``NativePagedResidency.write_native_paged_records``."""
        if local_device_after_commit and not self.supports_local_native_current_publication:
            raise ValueError("local current publication needs native paged storage on a GPU")
        fn = self._capability("write_native_paged_records", "bind record_storage_backend='native_paged'")
        if local_device_after_commit:
            return fn(layer, ids, source_record_pages, source_record_indices, local_device_after_commit=True)
        return fn(layer, ids, source_record_pages, source_record_indices)

    def _inputs_for_rows(self, layer: int, device_rows) -> ResidentAttentionInputs:
        from dataclasses import replace

        engine = self._live()
        planes = (engine.get_device_record_planes(layer) if hasattr(engine, "get_device_record_planes")
                  else tuple(engine.layer_plane(layer, p) for p in range(len(engine.planes))))
        template = ResidentAttentionInputs(record_planes=tuple(planes), device_record_indices=device_rows,
                                           records_per_page=self.cache_specification.storage_layout.records_per_page)
        return replace(template, pool_view=planes[0] if len(planes) == 1 else None)

    def prepare_prefill_attention_inputs(self, layer: int, selected_ids) -> ResidentAttentionInputs:
        """Eager prefill: the union of the selection becomes resident, the selection comes back as device rows."""
        rows = self._capability("plan_prefill", "prefill on this backend goes through the prefill windows")(layer, selected_ids)
        return self._inputs_for_rows(layer, rows)

    def prepare_prefill_record_chunk(self, layer: int, ids) -> ResidentAttentionInputs:
        """Borrow one bounded chunk of records (for reconstruction into the caller's workspace)."""
        rows = self._capability("prepare_prefill_record_chunk", "no borrowed-chunk interface")(layer, ids)
        return self._inputs_for_rows(layer, rows)

    def finish_prefill_record_chunk(self, layer: int):
        self._capability("finish_prefill_record_chunk", "no borrowed-chunk interface")(layer)

    def bind_prefill_reader(self, reader):
        """Attach the windowed prefill reader (``cache.prefill.window.WindowedPrefillReader``) that serves the three
        ``*_native_prefill_*`` calls of a tensor-parallel pool."""
        self._prefill_reader = reader

    def _reader(self):
        reader = getattr(self, "_prefill_reader", None)
        if reader is None:
            raise NotImplementedError("no windowed prefill reader is bound: this backend uses its resident chunk interface")
        return reader

    def prepare_native_prefill_read_plan(self, selected_ids):
        """Window plan of a prefill selection (no KV is read)."""
        return self._reader().prepare_read_plan(selected_ids)

    def read_native_prefill_records(self, layer: int, selected_ids, native_reader, *, output, read_plan=None):
        """Run the caller's reader over the bounded windows of the selection; it gets borrowed pages and remapped ids."""
        return self._reader().read_records(layer, selected_ids, native_reader, output_buffer=output, read_plan=read_plan)

    def attend_native_prefill_records(self, layer: int, query, selected_ids, lengths, native_attention):
        """Hand whole query windows to the caller's attention; selection and causal length stay paired per query."""
        return self._reader().attend(layer, query, selected_ids, lengths, native_attention)

    def offload_prefill_records(self, residency_group: int, ids):
        """Move a finished prefill's records of one residency group to the host tier."""
        import inspect

        fn = self._capability("offload_prefill", "this backend keeps prefill records where they were written")
        return fn(residency_group, ids) if len(inspect.signature(fn).parameters) >= 2 else fn(ids)

    def finish_layer_attention(self, layer: int):
        self._access.finish_layer(layer)

    def finish_model_forward(self):
        self._access.finish_forward()

    def abort_model_forward(self):
        self._access.abort_forward()

    def gather_selected_records(self, layer: int):
        """Dense uint8 ``[queries * width, record_bytes]`` copy of the prepared selection."""
        return self._live().gather_window(layer)

    # ------------------------------------------------------------- inventories --
    def memory_inventory(self) -> dict:
        return self._live().memory_inventory()

    def storage_inventory(self) -> dict:
        return self._live().storage_inventory()

    def get_memory_inventory(self) -> dict:
        return self.memory_inventory()

    def get_device_storage_inventory(self) -> dict:
        """Backing device allocations by address -> bytes, each counted once."""
        engine = self._live()
        if hasattr(engine, "device_storage_inventory"):
            return engine.device_storage_inventory()
        out = {}
        for st in engine.storages:
            storage = st.gpu.untyped_storage()
            out[storage.data_ptr()] = storage.nbytes()
        return out

    def get_host_storage_inventory(self) -> dict:
        """Pinned host allocations by address -> bytes, each counted once."""
        engine = self._live()
        if hasattr(engine, "host_storage_inventory"):
            return engine.host_storage_inventory()
        out = {}
        for st in engine.storages:
            if st.host is not None:
                storage = st.host.untyped_storage()
                out[storage.data_ptr()] = storage.nbytes()
        return out

    def get_device_record_planes(self, layer: int):
        """Every device plane of ``layer`` (borrowed; geometry is in the specification)."""
        engine = self._live()
        if hasattr(engine, "get_device_record_planes"):
            return engine.get_device_record_planes(layer)
        return tuple(engine.layer_plane(layer, p) for p in range(len(engine.planes)))

    @property
    def device_record_storage(self):
        """The single device plane ``[layers, slots, record_bytes]``; several planes: ``get_device_record_planes``."""
        engine = self._live()
        if len(engine.planes) != 1:
            raise ValueError("several planes are bound; use get_device_record_planes")
        return engine.gpu

    def counters(self) -> dict:
        return self._live().counters()

    def check(self, what="cache"):
        self._live().check(what)

    @property
    def engine(self):
        return self._engine

    def close(self):
        if self._engine is None:
            return
        self._access.require_idle("closing the cache")
        self._engine.close()
        self._slots.detach()
        self._engine = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


UlaCache = UnifiedMemoryCache
