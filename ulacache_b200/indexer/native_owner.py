"""Owner-side Index scoring over peer memory for ranks with independent queries.

Every rank asks about its own requests; the Index of every request is striped over all ranks
(logical page ``p`` on rank ``p % ranks``).  One call is

    export (peer stores) -> flag barrier -> index_score + top-k over world x rows queries on my shard
    -> return (peer stores, owner-local columns -> logical tokens) -> flag barrier -> merge top-k

with no library collective.  :class:`indexer.scorer.OwnerIndexScorer` is the same protocol composed
from ``all_gather`` calls; the two return the same selections (tests compare them).

Reference: ulacache/indexer/native_owner.py:153-477 (export / collect / score / restore over IPC
with three-phase flags), ulacache/indexer/kernels/scoring.py:83-984.
"""
from __future__ import annotations

import ctypes as C

from .ownership import IndexOwnership
from .plan import IndexScorePlan


class PeerOwnerIndexScorer:
    """``plan.rows`` = queries rows per rank (every rank passes that many; pad with length 0)."""

    def __init__(self, heap, plan: IndexScorePlan, *, n_q: int = 1, name: str = "owner_index"):
        import torch

        self.heap, self.plan, self.rank, self.world, self.n_q = heap, plan, heap.rank, heap.world, n_q
        if plan.ranks != self.world:
            raise ValueError("the plan's ranks must be the heap's world size")
        self.own = IndexOwnership(plan.ranks, plan.page_tokens)
        rows = plan.rows
        self.pages = (plan.local_columns + plan.page_tokens - 1) // plan.page_tokens
        w = self.world
        # inbox components, one slot per asker; double buffered by call parity
        shapes = [((w, rows, n_q, 64, 128), torch.uint8), ((w, rows, n_q, 64), torch.float32),
                  ((w, (rows + 3) // 4 * 4), torch.int32), ((w, rows, self.pages), torch.int32)]
        self.inbox = [[heap.alloc(f"{name}.in{p}.{c}", s, dt) for c, (s, dt) in enumerate(shapes)] for p in (0, 1)]
        self._slot_bytes = [t[0].numel() * t.element_size() for t in self.inbox[0]]
        for sb in self._slot_bytes:
            if sb % 16:
                raise ValueError("inbox slots must be multiples of 16 bytes (rows x pages x 4 for the table)")
        R = rows * n_q
        self.cand_v = [heap.alloc(f"{name}.cv{p}", (R, w, plan.topk), torch.float32) for p in (0, 1)]
        self.cand_t = [heap.alloc(f"{name}.ct{p}", (R, w, plan.topk), torch.int32) for p in (0, 1)]
        self._in_dst = [[heap.peer_ptr(r, t) for r in range(w) for t in self.inbox[p]] for p in (0, 1)]
        self._cv_dst = [heap.peer_ptrs(self.cand_v[p]) for p in (0, 1)]
        self._ct_dst = [heap.peer_ptrs(self.cand_t[p]) for p in (0, 1)]
        self.parity = 0
        self.bytes_exported_per_call = 0
        self.bytes_returned_per_call = 0

    def score(self, q8, w, page_table, lengths, pool, *, status=None):
        """``q8`` uint8 [rows, n_q, 64, 128], ``w`` fp32 [rows, n_q, 64], ``page_table`` int32
        [ranks (owner), rows, pages] (this rank's requests as every owner stores them, owner-local
        page numbers), ``lengths`` int32 [rows] logical lengths -> logical token positions int32
        [rows * n_q, topk] (-1 padded)."""
        import torch
        from ..ops import _native as N
        from ..ops import indexer, topk as topk_op

        p, plan, world = self.parity, self.plan, self.world
        rows, n_q, k = plan.rows, self.n_q, plan.topk
        if q8.shape[0] != rows or page_table.shape != (world, rows, self.pages):
            raise ValueError("every rank passes plan.rows query rows and a [ranks, rows, pages] table")
        q8, w, page_table = q8.contiguous(), w.contiguous().float(), page_table.contiguous()
        lens = torch.zeros((rows + 3) // 4 * 4, dtype=torch.int32, device=q8.device)
        lens[:rows] = lengths
        srcs = [q8, w, lens, page_table]
        nbytes = [q8.numel(), w.numel() * 4, lens.numel() * 4, rows * self.pages * 4]
        src_arr = (C.c_void_p * 4)(*[t.data_ptr() for t in srcs])
        by_arr = (C.c_longlong * 4)(*nbytes)
        slot_arr = (C.c_longlong * 4)(*self._slot_bytes)
        dst_arr = (C.c_void_p * (4 * world))(*self._in_dst[p])
        N.check(N.cuda().ulc_owner_export(src_arr, by_arr, slot_arr, dst_arr, C.c_int(self.rank), C.c_int(world),
                                          N.stream()), "owner_export")
        self.bytes_exported_per_call = sum(nbytes) * (world - 1)
        self.heap.device_barrier()
        # every asker's queries against my shard, one launch
        in_q, in_w, in_len, in_tab = self.inbox[p]
        all_len = in_len[:, :rows].reshape(world * rows)
        scores = indexer.index_score(in_q.view(world * rows, n_q, 64, 128), in_w.view(world * rows, n_q, 64),
                                     in_tab.view(world * rows, self.pages), all_len, pool, ranks=world, rank=self.rank,
                                     status=status)
        local_len = self.own.local_length(all_len, self.rank).to(torch.int32)
        if n_q > 1:
            local_len = local_len.repeat_interleave(n_q)
        R = rows * n_q
        vals = torch.empty((world * R, k), dtype=torch.float32, device=q8.device)
        cols = topk_op.topk(scores, k, lengths=local_len.contiguous(), out_val=vals)
        cv = (C.c_void_p * world)(*self._cv_dst[p])
        ct = (C.c_void_p * world)(*self._ct_dst[p])
        N.check(N.cuda().ulc_owner_return(N.ptr(vals), N.ptr(cols), cv, ct, C.c_int(self.rank), C.c_int(world),
                                          C.c_int(R), C.c_int(k), C.c_int(plan.page_tokens), N.stream()), "owner_return")
        self.bytes_returned_per_call = R * k * 8 * (world - 1)
        self.heap.device_barrier()
        self.parity ^= 1
        return topk_op.topk(self.cand_v[p].view(R, world * k), k, in_idx=self.cand_t[p].view(R, world * k))
