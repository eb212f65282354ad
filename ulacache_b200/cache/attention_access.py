"""Framework-agnostic ordering of one tier's calls around a model forward.

A serving framework drives the cache through five moments; this class checks their order and
forwards them to a cache client:

    begin(batch)                              once per forward
      per layer: prepare(layer, selection, current) -> publish(layer, values) -> view(layer)
                 ... attention ...            -> finish_layer(layer)
    finish()                                  once per forward (abort() on an exception)

Reference: ulacache/cache/attention_access.py:6-263 (NativeSparseCacheExecution).
"""
from __future__ import annotations

from .access import SparseAttentionAccessPlan


class LifecycleError(RuntimeError):
    pass


class NativeSparseCacheExecution:
    def __init__(self, client, layer_count: int):
        self.client, self.layer_count = client, layer_count
        self._open = False
        self._layer_state = {}

    def begin(self, context=None):
        if self._open:
            raise LifecycleError("forward already open")
        self.client.begin_model_forward(context)
        self._open = True
        self._layer_state = {}

    def _need_open(self):
        if not self._open:
            raise LifecycleError("no forward is open")

    def prepare(self, layer: int, selection, current=None):
        self._need_open()
        if not 0 <= layer < self.layer_count:
            raise LifecycleError(f"layer {layer} out of range")
        if self._layer_state.get(layer) not in (None, "finished"):
            raise LifecycleError(f"layer {layer} prepared twice")
        self.client.prepare_sparse_attention(layer, SparseAttentionAccessPlan(selection, current))
        self._layer_state[layer] = "prepared"

    def publish(self, layer: int, ids, values):
        self._need_open()
        if self._layer_state.get(layer) != "prepared":
            raise LifecycleError(f"layer {layer}: publish before prepare")
        self.client.write(ids, layer, values)
        self._layer_state[layer] = "published"

    def view(self, layer: int):
        self._need_open()
        if self._layer_state.get(layer) not in ("prepared", "published"):
            raise LifecycleError(f"layer {layer}: view before prepare")
        self._layer_state[layer] = "reading"
        return self.client.get_resident_attention_inputs(layer)

    def finish_layer(self, layer: int):
        self._need_open()
        if self._layer_state.get(layer) != "reading":
            raise LifecycleError(f"layer {layer}: finish before view")
        self.client.finish_layer_attention(layer)
        self._layer_state[layer] = "finished"

    def finish(self):
        self._need_open()
        live = [l for l, s in self._layer_state.items() if s == "reading"]
        if live:
            raise LifecycleError(f"layers {live} still have live views")
        self.client.finish_model_forward()
        self._open = False

    def abort(self):
        if self._open:
            self.client.abort_model_forward()
            self._open = False
            self._layer_state = {}


# ----------------------------------------------------------------------------------------------
# The fuller adapter a serving framework binds: writer staging, decode and prefill paths, chunked
# reconstruction of prefix records, page-granular registration, inventories.
#
# Reference: ulacache/cache/attention_access.py:14-263 (begin_forward, prepare_attention with the
# pending-current logic, reconstruct_prefill_records, finish_attention, register_full_pages /
# release_full_pages / clear_records, get_device_storage_inventory).
# ----------------------------------------------------------------------------------------------
class WriterStaging:
    """What the model's KV writer produced for a layer and has not yet published to the cache: logical ids and
    either encoded records (uint8 [n, record_bytes]) or (latent, rope) tensors."""

    def __init__(self):
        self._staged = {}
        self.published_records = 0

    def stage(self, layer: int, ids, values):
        if ids.dim() != 1:
            raise ValueError("staged ids are one-dimensional")
        self._staged[layer] = (ids, values)

    def pending_logical_record_ids(self, layer: int):
        item = self._staged.get(layer)
        return None if item is None else item[0]

    def publish_staged_records(self, client, layer: int, *, local_device_after_commit: bool = False):
        item = self._staged.pop(layer, None)
        if item is None:
            return 0
        ids, values = item
        engine = getattr(client, "engine", None)
        if local_device_after_commit and hasattr(engine, "write_native_paged_records") and values.__class__.__name__ == "Tensor":
            import torch

            engine.write_native_paged_records(layer, ids, values, torch.arange(ids.numel(), device=values.device),
                                              local_device_after_commit=True)
        else:
            client.write(ids, layer, values)
        self.published_records += int(ids.numel())
        return int(ids.numel())

    def get_device_storage_inventory(self) -> dict:
        inv = {}
        for ids, values in self._staged.values():
            for t in (ids,) + (tuple(values) if isinstance(values, tuple) else (values,)):
                if hasattr(t, "untyped_storage"):
                    inv[t.untyped_storage().data_ptr()] = t.untyped_storage().nbytes()
        return inv


class FrameworkCacheExecution(NativeSparseCacheExecution):
    """``client``: a :class:`~ulacache_b200.client.UnifiedMemoryCache`.  Decode-like forwards (decode, verify)
    run the residency transaction per selection producer with the writer's pending ids as the current records;
    prefill forwards go through the request-group buffers when given, else through the engine's eager union."""

    def __init__(self, client, layer_count: int, *, device, query_capacity: int, records_per_page: int = 64,
                 prefill_chunk_capacity=None, prefill_buffers=None, writer_staging=None,
                 local_current_publication: bool = False):
        import torch

        super().__init__(client, layer_count)
        if type(local_current_publication) is not bool:
            raise ValueError("local current publication must be explicitly boolean")
        self.device, self.records_per_page = device, records_per_page
        self.query_capacity = query_capacity
        spec = client.cache_specification
        self.prefill_chunk_capacity = prefill_chunk_capacity or spec.capacity_plan.device_record_capacity
        self.prefill_buffers = prefill_buffers
        self.writer_staging = writer_staging or WriterStaging()
        self.local_current_publication = local_current_publication
        self.groups = spec.layer_reuse.residency_groups()
        self.current_write_records = torch.full((query_capacity,), -1, dtype=torch.int32, device=device)
        self.no_current_write_records = torch.full_like(self.current_write_records, -1)
        # records 1 .. page - 1 of the first page are never handed out: register them so that padded page tables
        # resolve to something allocated
        self.reserved_logical_records = torch.arange(1, records_per_page, dtype=torch.int32, device=device)
        self.decode_like = False
        self._resident_prefill_layers = set()
        self._committed_current = {}

    # ------------------------------------------------------------------- forward --
    def begin_forward(self, *, decode_like: bool, query_count: int, prefill_request_query_counts=None, context=None):
        if query_count > self.query_capacity:
            raise ValueError("more queries than the startup bound")
        self.decode_like = decode_like
        self.query_count = query_count
        if self.prefill_buffers is not None:
            self.prefill_buffers.begin_forward(None if decode_like else prefill_request_query_counts)
        self._resident_prefill_layers.clear()
        self._committed_current = {}
        self.begin(context)

    def publish_after_native_write(self, layer: int):
        """Prefill: the writer's records are published as soon as they exist (decode publishes inside
        ``prepare_attention``, after the transaction that makes room for them)."""
        if not self.decode_like:
            self.writer_staging.publish_staged_records(self.client, layer)

    def prepare_attention(self, layer: int, logical_record_ids):
        """Returns the selection as device rows (decode, eager prefill) or as given (request-group prefill, where
        the buffers rewrite it group by group), shaped like ``logical_record_ids``."""
        import torch

        self._need_open()
        shape = logical_record_ids.shape
        selected = logical_record_ids.flatten(1).to(torch.int32).contiguous()
        q = shape[0]
        g = self.groups.group(layer)
        if self.decode_like:
            pending = self.writer_staging.pending_logical_record_ids(layer)
            if self.groups.anchors[g] == layer:
                current = self.no_current_write_records[:q]
                if pending is not None:
                    if pending.numel() == q:
                        current = pending.to(torch.int32)
                    else:                                   # padded batch: the tail stays -1
                        self.current_write_records.fill_(-1)
                        self.current_write_records[: pending.numel()].copy_(pending)
                        current = self.current_write_records[:q]
                self.prepare(layer, selected, current)
                engine = getattr(self.client, "engine", None)
                if (self.local_current_publication and pending is not None and pending.numel() <= q
                        and getattr(engine, "supports_local_native_current_publication", False) is True):
                    # the transaction has just made every current record device-resident here
                    self._committed_current[g] = (pending.data_ptr(), tuple(pending.shape))
            else:
                self._layer_state[layer] = "prepared"       # a follower reuses its anchor's plan
            if pending is not None:                          # a follower can still own its own KV payload
                committed = self._committed_current.get(g)
                local = committed is not None and committed == (pending.data_ptr(), tuple(pending.shape))
                self.writer_staging.publish_staged_records(self.client, layer, local_device_after_commit=local)
            inputs = self.view(layer)
            return inputs.device_record_indices.reshape(shape)
        if self.prefill_buffers is not None:
            return self.prefill_buffers.select(layer, selected).reshape(shape)
        engine = self.client.engine
        rows = engine.plan_prefill(layer, selected)
        self._resident_prefill_layers.add(layer)
        self._layer_state[layer] = "reading"
        return rows.reshape(shape)

    def reconstruct_prefill_records(self, layer: int, logical_record_ids, output, read_native_records):
        """Rebuild a prefix in ``output`` (one tensor or a tuple of planes, first dimension = records) chunk by
        chunk: ``read_native_records(record_planes, device_rows, output_chunk)``."""
        engine = self.client.engine
        n = int(logical_record_ids.numel())
        for start in range(0, n, self.prefill_chunk_capacity):
            stop = min(start + self.prefill_chunk_capacity, n)
            rows = engine.prepare_prefill_record_chunk(layer, logical_record_ids[start:stop])
            chunk = tuple(p[start:stop] for p in output) if isinstance(output, tuple) else output[start:stop]
            try:
                read_native_records(engine.get_device_record_planes(layer), rows, chunk)
            finally:
                engine.finish_prefill_record_chunk(layer)

    def finish_attention(self, layer: int):
        if self.decode_like:
            self.finish_layer(layer)
            g = self.groups.group(layer)
            if self.groups.layers_of(g)[-1] == layer:
                self._committed_current.pop(g, None)
        elif layer in self._resident_prefill_layers:
            self.client.engine.after_attention(layer)
            self._resident_prefill_layers.discard(layer)
            self._layer_state[layer] = "finished"

    # --------------------------------------------------------------------- pages --
    def _records_of_pages(self, page_ids):
        import torch

        return (page_ids.reshape(-1, 1).long() * self.records_per_page
                + torch.arange(self.records_per_page, device=page_ids.device)).reshape(-1).to(torch.int32)

    def register_full_pages(self, page_ids, *, prefer_device: bool):
        """Whole pages at once (unwritten page tails are masked by the causal lengths anyway)."""
        self.client.register_logical_records(self._records_of_pages(page_ids), prefer_device=prefer_device)

    def release_full_pages(self, page_ids):
        self.client.release_logical_records(self._records_of_pages(page_ids))

    def register_reserved_records(self):
        self.client.register_logical_records(self.reserved_logical_records)

    def clear_records(self):
        self._committed_current.clear()
        self.client.clear_registered_records()
        self.register_reserved_records()

    def get_device_storage_inventory(self) -> dict:
        engine = self.client.engine
        inv = dict(engine.device_storage_inventory()) if hasattr(engine, "device_storage_inventory") else {}
        inv.update(self.writer_staging.get_device_storage_inventory())
        for t in (self.current_write_records, self.no_current_write_records, self.reserved_logical_records):
            inv[t.untyped_storage().data_ptr()] = t.untyped_storage().nbytes()
        if self.prefill_buffers is not None:
            inv.update(self.prefill_buffers.inventory())
        return inv
