"""Index score transports: how the ranks' partial index scores (or top-k candidates) meet.

    transport = create_index_transport("candidates" | "tagged" | "nccl", ...)
    all_scores = transport.all_gather_scores(local)        # [ranks, rows, local_cols]

* ``tagged``   - :class:`LineScoreAllGather`: barrier-free all-gather through peer memory in 128-byte
  lines of 31 payload words + 1 tag word (96.9 % wire efficiency), ragged rows packed on the wire with
  their device-side lengths in header lines (kernel ``line_all_gather_kernel``).
* ``tagged_words`` - :class:`TaggedScoreAllGather`: the simpler wire format, every 8-byte word carries
  4 payload bytes and its call index (kernel ``tagged_all_gather_kernel``); kept for comparison.
* ``nccl``     - :class:`CollectiveScoreAllGather`: ``all_gather_into_tensor`` (NCCL on GPUs, gloo on
  CPU ranks); the baseline.
* ``candidates`` is not an all-gather at all: ranks exchange their local top-k candidates
  (``parallel.peer_collectives.PeerCandidateExchange``); ``create_index_transport`` returns the
  exchange object for it.

Unlike the reference, compute capability (10, 0) is accepted: nothing here depends on NVLS
multicast or on sm_103.

Reference: ulacache/flashag/__init__.py:70-101 (create_index_owner, capability gate),
owner.py:219, packed.py:91-93 (local column count), b300_layout.py (slab layout).
"""
from __future__ import annotations

import ctypes as C
from abc import ABC, abstractmethod
from dataclasses import dataclass

AG_SLOTS = 4


def local_columns(width: int, world: int) -> int:
    """Columns of one rank's score slice for a logical score width ``width``: the rank's share,
    rounded up to 64-token pages and then to 256 columns (whole 1 KiB fp32 lines per row)."""
    share = (width + world - 1) // world
    return (share + 255) // 256 * 256


@dataclass(frozen=True)
class SlabLayout:
    """Receive slab of the tagged all-gather on every rank: [slot][source rank][row words] of
    8-byte (value, tag) words."""

    world: int
    max_words: int              # fp32 words one rank contributes per call (rows * local_cols)
    slots: int = AG_SLOTS

    @property
    def bytes(self) -> int:
        return self.slots * self.world * self.max_words * 8

    def word_offset(self, slot: int, source: int) -> int:
        return (slot * self.world + source) * self.max_words


LINE_WORDS = 31            # payload words of a 128-byte line; word 31 is the call index


def line_count(rows: int, cols: int) -> int:
    """Lines of one rank's message at most: header (payload length + one length per row) + payload."""
    return (rows + 1 + LINE_WORDS - 1) // LINE_WORDS + (rows * cols + LINE_WORDS - 1) // LINE_WORDS


@dataclass(frozen=True)
class LineSlabLayout:
    """Receive slab of the line all-gather on every rank: [slot][source rank][lines] of 128 bytes."""

    world: int
    max_lines: int
    slots: int = AG_SLOTS

    @property
    def bytes(self) -> int:
        return self.slots * self.world * self.max_lines * 128

    def line_offset(self, slot: int, source: int) -> int:
        return (slot * self.world + source) * self.max_lines

    @staticmethod
    def wire_efficiency() -> float:
        return LINE_WORDS / 32.0


def pack_lines(rows, lens, tag: int):
    """Host model of one message (numpy): fp32 ``rows`` [R, C] with valid prefixes ``lens`` -> uint32
    [lines, 32].  The kernel and this function must agree; tests compare them through unpack_lines."""
    import numpy as np

    rows = np.asarray(rows, dtype=np.float32)
    lens = np.clip(np.asarray(lens, dtype=np.int64), 0, rows.shape[1])
    payload = np.concatenate([rows[r, : lens[r]] for r in range(rows.shape[0])]) if rows.shape[0] else np.zeros(0, np.float32)
    header = np.concatenate([[payload.size], lens]).astype(np.uint32)
    out = []
    for words in (header, payload.view(np.uint32)):
        n = (words.size + LINE_WORDS - 1) // LINE_WORDS
        padded = np.zeros(n * LINE_WORDS, dtype=np.uint32)
        padded[: words.size] = words
        buf = np.zeros((n, 32), dtype=np.uint32)
        buf[:, :LINE_WORDS] = padded.reshape(n, LINE_WORDS)
        buf[:, LINE_WORDS] = tag
        out.append(buf)
    return np.concatenate(out)


def unpack_lines(lines, n_rows: int, cols: int, tag: int, fill: float):
    """Inverse of :func:`pack_lines`; raises when a line's tag is not ``tag``."""
    import numpy as np

    lines = np.asarray(lines, dtype=np.uint32)
    header_lines = (n_rows + 1 + LINE_WORDS - 1) // LINE_WORDS
    header = np.ascontiguousarray(lines[:header_lines, :LINE_WORDS]).reshape(-1)
    total, lens = int(header[0]), header[1: n_rows + 1].astype(np.int64)
    n_payload = (total + LINE_WORDS - 1) // LINE_WORDS
    used = lines[: header_lines + n_payload]
    if not (used[:, LINE_WORDS] == tag).all():
        raise ValueError("a line of the message carries another call's tag")
    payload = np.ascontiguousarray(used[header_lines:, :LINE_WORDS]).reshape(-1)[:total].view(np.float32)
    out = np.full((n_rows, cols), fill, dtype=np.float32)
    at = 0
    for r in range(n_rows):
        out[r, : lens[r]] = payload[at: at + lens[r]]
        at += lens[r]
    return out, lens


class IndexTransport(ABC):
    world: int
    rank: int

    @abstractmethod
    def all_gather_scores(self, local):
        """``local`` fp32 [rows, cols] -> fp32 [world, rows, cols] in rank order."""

    def close(self):
        pass


class CollectiveScoreAllGather(IndexTransport):
    def __init__(self, group, rank: int, world: int):
        self.group, self.rank, self.world = group, rank, world

    def all_gather_scores(self, local):
        import torch
        import torch.distributed as dist

        local = local.contiguous()
        out = torch.empty((self.world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
        if self.world == 1:
            out[0] = local
            return out
        if local.is_cuda:
            dist.all_gather_into_tensor(out, local, group=self.group)
        else:
            parts = [torch.empty_like(local) for _ in range(self.world)]
            dist.all_gather(parts, local, group=self.group)
            out = torch.stack(parts)
        return out


class TaggedScoreAllGather(IndexTransport):
    def __init__(self, heap, max_rows: int, cols: int, name: str = "score_ag", limit_cycles: int = 0):
        import torch

        self.heap, self.rank, self.world = heap, heap.rank, heap.world
        self.layout = SlabLayout(self.world, max_rows * cols)
        self.slab = heap.alloc(name, (self.layout.bytes // 8,), torch.int64)
        self.slab.zero_()
        self._slabs = heap.peer_ptrs(self.slab)
        self.counter = torch.zeros(2, dtype=torch.int32, device=heap.device)
        self.limit = limit_cycles
        import torch.distributed as dist

        if self.world > 1:
            dist.barrier(group=heap.cpu_group)          # every slab is zeroed before anyone sends

    def all_gather_scores(self, local):
        import torch
        from ..ops import _native as N

        local = local.contiguous()
        n = local.numel()
        out = torch.empty((self.world,) + tuple(local.shape), dtype=torch.float32, device=local.device)
        arr = (C.c_void_p * self.world)(*self._slabs)
        N.check(N.cuda().ulc_tagged_all_gather(N.ptr(local), C.c_int(n), C.c_int(self.layout.max_words), arr,
                                               C.c_int(self.rank), C.c_int(self.world), N.ptr(self.counter),
                                               N.ptr(out), C.c_longlong(self.limit), N.ptr(self.heap.status),
                                               N.stream()), "tagged_all_gather")
        return out


def line_all_gather_raw(local, row_len, slab_ptrs, rank: int, world: int, max_lines: int, slots: int, counter, status,
                        *, fill: float = float("-inf"), out=None, out_len=None, max_ctas: int = 0, limit_cycles: int = 0):
    """One launch of ``line_all_gather_kernel``.  ``slab_ptrs``: device addresses of every rank's
    receive slab (``slots * world * max_lines`` lines, zeroed before the first call); ``counter``
    device int32[2] (zeroed).  -> (fp32 [world, rows, cols], int32 [world, rows])."""
    import torch
    from ..ops import _native as N

    rows, cols = local.shape
    if out is None:
        out = torch.empty((world, rows, cols), dtype=torch.float32, device=local.device)
    if out_len is None:
        out_len = torch.empty((world, rows), dtype=torch.int32, device=local.device)
    arr = (C.c_void_p * world)(*slab_ptrs)
    N.check(N.cuda().ulc_line_all_gather(
        N.ptr(local), C.c_longlong(local.stride(0)), N.ptr(row_len), C.c_int(rows), C.c_int(cols), arr, C.c_int(rank),
        C.c_int(world), C.c_int(max_lines), C.c_int(slots), N.ptr(counter), N.ptr(out), N.ptr(out_len), C.c_float(fill),
        C.c_int(max_ctas), C.c_longlong(limit_cycles), N.ptr(status), N.stream()), "line_all_gather")
    return out, out_len


class LineScoreAllGather(IndexTransport):
    """All-gather of fp32 rows [rows, cols] (optionally ragged: ``row_len`` device int32 [rows]) over the
    symmetric heap in tagged 128-byte lines.  No barrier and no host-side length: a receiver learns
    each sender's payload length from the sender's header lines."""

    def __init__(self, heap, max_rows: int, cols: int, name: str = "line_ag", limit_cycles: int = 0,
                 slots: int = AG_SLOTS, max_ctas: int = 0):
        import torch
        import torch.distributed as dist

        if max_rows > 4096:
            raise ValueError("at most 4096 rows per message")
        self.heap, self.rank, self.world = heap, heap.rank, heap.world
        self.max_rows, self.cols = max_rows, cols
        self.layout = LineSlabLayout(self.world, line_count(max_rows, cols), slots)
        self.slab = heap.alloc(name, (self.layout.bytes // 8,), torch.int64)
        self.slab.zero_()
        self._slabs = heap.peer_ptrs(self.slab)
        self.counter = torch.zeros(2, dtype=torch.int32, device=heap.device)
        self.limit, self.max_ctas = limit_cycles, max_ctas
        if self.world > 1:
            dist.barrier(group=heap.cpu_group)          # every slab is zeroed before anyone sends

    def all_gather(self, local, row_len=None, fill: float = float("-inf"), out=None, out_len=None):
        """-> (fp32 [world, rows, cols], int32 [world, rows] valid lengths)."""
        import torch
        from ..ops import _native as N

        rows, cols = local.shape
        if cols != self.cols or rows > self.max_rows or local.stride(1) != 1 or local.dtype != torch.float32:
            raise ValueError("rows of fp32 with the configured width expected")
        return line_all_gather_raw(local, row_len, self._slabs, self.rank, self.world, self.layout.max_lines,
                                   self.layout.slots, self.counter, self.heap.status, fill=fill, out=out,
                                   out_len=out_len, max_ctas=self.max_ctas, limit_cycles=self.limit)

    def all_gather_scores(self, local):
        return self.all_gather(local.contiguous().view(-1, self.cols) if local.dim() != 2 else local)[0].view(
            (self.world,) + tuple(local.shape))


def create_index_transport(kind: str, *, heap=None, group=None, rank: int = 0, world: int = 1, max_rows: int = 0,
                           cols: int = 0, topk: int = 0, device=None, cpu_group=None):
    """``kind``: "candidates" (peer-stored top-k candidates, the default product path), "tagged"
    (barrier-free score all-gather in 128-byte lines), "tagged_words" (8-byte words) or "nccl"
    (library all-gather; with ``device`` and the bounds ``max_rows`` x ``cols`` local columns it is the
    workspace-owning form that a captured graph can replay)."""
    if kind == "nccl" or (kind in ("tagged", "tagged_words") and heap is None):
        if kind == "nccl" and device is not None and max_rows > 0 and cols > 0 and cols % 64 == 0:
            from ..indexer.nccl import CollectiveIndexOwner

            return CollectiveIndexOwner(group, rank=rank, world=world, max_queries=max_rows,
                                        max_page_width=cols // 64 * world, device=device, cpu_group=cpu_group)
        return CollectiveScoreAllGather(group, rank, world)
    if kind == "tagged":
        return LineScoreAllGather(heap, max_rows, cols)
    if kind == "tagged_words":
        return TaggedScoreAllGather(heap, max_rows, cols)
    if kind == "candidates":
        from ..parallel.peer_collectives import PeerCandidateExchange

        if heap is None:
            raise ValueError("the candidate exchange needs a symmetric heap")
        return PeerCandidateExchange(heap, max_rows, topk)
    raise ValueError(f"unknown index score transport {kind!r}")
