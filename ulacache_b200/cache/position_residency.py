"""Context-parallel (position-sharded) wrapper around a rank-local engine.

Global slot ``s`` lives on rank ``s % CP`` as local slot ``s // CP``.  Each rank
keeps, per query, only the selected slots it holds (compacted to the front, with a
per-query count), runs attention over those, and the partial outputs are merged
by log-sum-exp weights (``merge_partial_attention``).

Reference: PositionShardedResidency (ulacache/cache/position_residency.py:11,
plan :112), the `_selection` kernel (ulacache/cache/kernels/position.py:8) and the
O/LSE all-to-all merge (patches/sglang.patch:1983-2011).
"""
from __future__ import annotations

from .access import SparseAttentionAccessPlan


def localize_selection(sel, ranks: int, rank: int):
    """Keep ``slot % ranks == rank``, convert to local slots, compact each row to the
    front.  Returns (int32 [Q, K] local IDs padded with 0, int32 [Q] counts)."""
    import torch

    keep = (sel > 0) & ((sel % ranks) == rank)
    local = torch.where(keep, sel // ranks, torch.zeros_like(sel))
    order = torch.argsort((~keep).to(torch.int8), dim=1, stable=True)
    return torch.gather(local, 1, order).to(torch.int32), keep.sum(dim=1).to(torch.int32)


def merge_partial_attention(outs, lses):
    """Merge per-rank partial attention: ``outs`` [R, Q, H, D], ``lses`` [R, Q, H]
    (natural-log sum-exp; -inf where a rank had nothing)."""
    import torch

    m = lses.max(dim=0).values
    w = torch.exp(lses - m.unsqueeze(0))
    w = torch.where(torch.isfinite(lses), w, torch.zeros_like(w))
    denom = w.sum(dim=0).clamp_min(1e-30)
    out = (outs * w.unsqueeze(-1)).sum(dim=0) / denom.unsqueeze(-1)
    return out, m + torch.log(denom)


class PositionShardedResidency:
    """Engine protocol adaptor: global ids in, local engine underneath.

    Everything a decode step touches lives in buffers allocated here once - the localised selection and its
    counts per residency group, the mapped current ids - so a captured step replays over stable addresses and
    allocates nothing; registration and release are eager allocator operations and may allocate.  The mapping of
    the step's current ids is cached by the identity of the tensor it was computed from (the same tensor is
    handed in for every layer of a forward)."""

    def __init__(self, inner, layout, rank: int, *, max_queries=None, topk=None):
        import torch

        self.inner, self.layout, self.rank = inner, layout, rank
        access = inner.spec.sparse_access
        self.max_queries = int(max_queries or access.maximum_padded_query_count)
        self.topk = int(topk or access.maximum_selected_record_count)
        opts = dict(dtype=torch.int32, device=inner.device)
        groups = inner.groups.group_count
        self.selected = torch.zeros((groups, self.max_queries, self.topk), **opts)
        self.selected_count = torch.zeros((groups, self.max_queries), **opts)
        self.current = torch.full((self.max_queries,), -1, **opts)
        self._current_signature = None
        self.counts = {}
        self._closed = False

    def __getattr__(self, name):
        return getattr(self.inner, name)

    # ------------------------------------------------------------------ mapping --
    def _local_ids(self, ids):
        import torch

        keep = (ids > 0) & ((ids % self.layout.ranks) == self.rank)
        return (ids[keep] // self.layout.ranks).to(torch.int32)

    @staticmethod
    def _signature(t):
        return (t.data_ptr(), t.numel(), t.dtype, getattr(t, "_version", 0))

    def _map_current(self, ids):
        """Per-query current ids (padded order kept): the local id where this rank owns the position, -1 elsewhere."""
        import torch

        sig = self._signature(ids)
        n = ids.numel()
        if self._current_signature != sig:
            flat = ids.reshape(-1)
            keep = (flat > 0) & ((flat % self.layout.ranks) == self.rank)
            self.current[:n].copy_(torch.where(keep, flat // self.layout.ranks, torch.full_like(flat, -1)).to(torch.int32))
            self._current_signature = sig
        return self.current[:n]

    # ----------------------------------------------------------------- lifetime --
    def allocate_unbound(self, ids, prefer_gpu=True):
        self.inner.allocate_unbound(self._local_ids(ids.reshape(-1)), prefer_gpu=prefer_gpu)

    def release(self, ids):
        self.inner.release(self._local_ids(ids.reshape(-1)))

    def begin_forward(self, context=None):
        self._current_signature = None
        self.inner.begin_forward(context)

    def begin_prefill(self, ids):
        """A prefill chunk may be wider than the decode bound: only a chunk that fits uses the step buffers."""
        self._current_signature = None
        if ids.numel() <= self.max_queries:
            self._map_current(ids)

    def finish_forward(self):
        self.inner.finish_forward()
        self._current_signature = None

    # --------------------------------------------------------------------- plan --
    def plan(self, layer, access: SparseAttentionAccessPlan):
        import torch

        sel = access.selected_logical_record_ids
        cur = access.current_logical_record_ids
        if sel.dim() != 2 or sel.shape[0] > self.max_queries or sel.shape[1] > self.topk:
            raise ValueError("the selection exceeds the fixed query / top-k bounds of the position-sharded engine")
        if cur is not None and cur.numel() != sel.shape[0]:
            raise ValueError("current records must keep the padded query order (one per query)")
        q, k = sel.shape
        g = self.inner.groups.group(layer)
        if sel.is_cuda:
            from ..ops import prefill as P

            local, counts = P.cp_localize(sel.to(torch.int32).contiguous(), self.layout.ranks, self.rank)
        else:
            local, counts = localize_selection(sel, self.layout.ranks, self.rank)
        dst = self.selected[g, :q, :k]
        dst.copy_(local)
        self.selected_count[g, :q].copy_(counts)
        self.counts[g] = self.selected_count[g, :q]
        mapped = None
        if cur is not None:
            m = self._map_current(cur)
            mapped = m[m > 0] if not sel.is_cuda else m          # (the CPU reference engine takes owned ids only)
        return self.inner.plan(layer, SparseAttentionAccessPlan(dst if k == self.topk else dst.contiguous(), mapped))

    def selected_counts(self, layer):
        return self.counts[self.inner.groups.group(layer)]

    def attention_rows(self, layer):
        # the rows are LOCAL physical rows already: the caller must not apply slot % CP / slot // CP again
        return self.inner.attention_rows(layer)

    def write(self, layer, ids, values, **kw):
        import torch

        flat = ids.reshape(-1)
        keep = (flat > 0) & ((flat % self.layout.ranks) == self.rank)
        if not bool(keep.any()):
            return
        if torch.is_tensor(values):
            vals = values[keep]
        else:
            vals = tuple(v[keep] for v in values)
        self.inner.write(layer, (flat[keep] // self.layout.ranks).to(torch.int32), vals, **kw)

    # --------------------------------------------------------------- unsupported --
    def allocate_receive_rows(self, ids):
        raise NotImplementedError("remote receive into a position-sharded cache needs an owner-aware transport binding")

    def plan_prefill(self, layer, selection):
        raise NotImplementedError("position-sharded prefill goes through the two-window materializer, not a resident union")

    # ---------------------------------------------------------------- inventory --
    def _mapping_tensors(self):
        return (self.selected, self.selected_count, self.current)

    def device_storage_inventory(self) -> dict:
        inv = dict(self.inner.device_storage_inventory()) if hasattr(self.inner, "device_storage_inventory") else {}
        for t in self._mapping_tensors():
            st = t.untyped_storage()
            inv[st.data_ptr()] = st.nbytes()
        return inv

    def host_storage_inventory(self) -> dict:
        return self.inner.host_storage_inventory() if hasattr(self.inner, "host_storage_inventory") else {}

    def memory_inventory(self) -> dict:
        inv = dict(self.inner.memory_inventory())
        extra = sum(t.numel() * t.element_size() for t in self._mapping_tensors())
        inv["metadata_bytes"] = inv.get("metadata_bytes", 0) + extra
        cap = self.inner.spec.capacity_plan
        inv.update(record_distribution="position_modulo_cp", storage_owner_rank=self.rank,
                   storage_owner_count=self.layout.ranks,
                   global_logical_record_capacity=cap.logical_record_capacity * self.layout.ranks,
                   peer_kv_read_bytes=0, replicated_decode_attention_payload_bytes=0, additional_mapping_bytes=extra)
        return inv

    def close(self):
        if self._closed:
            return
        self.inner.close()
        self.selected = self.selected_count = self.current = None
        self._closed = True
