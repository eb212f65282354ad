"""Selection-address trace: a bounded device ring of (step, layer, record id) triples that the
decode step appends to, drained to the host in chunks between steps and saved as ``.npy``.

A chunk that would overflow the ring is dropped whole and counted (the step is never stalled).

Reference: ulacache/telemetry/sparse_trace.py:74 (GpuSparseTraceRecorder), tp_sparse_trace.py:4.
"""
from __future__ import annotations

import ctypes as C


class GpuSparseTraceRecorder:
    def __init__(self, device, capacity_triples: int = 1 << 22):
        import torch

        self.capacity = int(capacity_triples)
        self.ring = torch.zeros((self.capacity, 3), dtype=torch.int32, device=device)
        self.header = torch.tensor([0, 0, self.capacity], dtype=torch.int64, device=device)
        self.chunks = []           # drained host chunks (int32 [n, 3])

    def record(self, step: int, layer: int, selection):
        import torch

        sel = selection.reshape(-1).to(torch.int32).contiguous()
        n = int(sel.numel())
        if self.ring.is_cuda:
            from ..ops import _native as N

            N.check(N.cuda().ulc_trace_append(N.ptr(self.ring), N.ptr(self.header), C.c_int(step), C.c_int(layer),
                                              N.ptr(sel), C.c_longlong(n), N.stream()), "trace_append")
            return
        cur = int(self.header[0])
        if cur + n > self.capacity:
            self.header[1] += n
            return
        self.ring[cur:cur + n, 0] = step
        self.ring[cur:cur + n, 1] = layer
        self.ring[cur:cur + n, 2] = sel
        self.header[0] = cur + n

    def drain(self):
        """Copy what was recorded to the host and rewind the ring.  Call between steps."""
        n = int(self.header[0])
        if n:
            self.chunks.append(self.ring[:n].cpu().numpy().copy())
        self.header[0] = 0
        return n

    @property
    def dropped(self) -> int:
        return int(self.header[1])

    def save(self, path: str):
        import numpy as np

        self.drain()
        data = np.concatenate(self.chunks) if self.chunks else np.zeros((0, 3), dtype=np.int32)
        np.save(path, data)
        return data.shape[0]


def load_trace(path: str):
    """Per (step, layer) lists of selected ids from a saved trace: {(step, layer): ndarray}."""
    import numpy as np

    data = np.load(path)
    out = {}
    if data.shape[0] == 0:
        return out
    key = data[:, 0].astype(np.int64) * (1 << 20) + data[:, 1]
    order = np.argsort(key, kind="stable")
    data, key = data[order], key[order]
    cuts = np.flatnonzero(np.diff(key)) + 1
    for chunk in np.split(data, cuts):
        out[(int(chunk[0, 0]), int(chunk[0, 1]))] = chunk[:, 2].copy()
    return out


# ------------------------------------------------------------------------------------------------------
# Framed capture: what a policy replay needs beyond the ids.  Every forward is one frame holding, per residency
# group, the selection of every query row, the record each row is writing (its "current" record, which is never
# a lookup), the group's epoch, and how many rows were valid; allocation and release of records are logged as
# events between frames.  Buffers are fixed at construction and written only by device-side ops whose target slot
# comes from a device scalar, so the observers can sit inside a captured CUDA graph; the host drains one chunk of
# frames at a time at a synchronising boundary that is kept out of any timed region.
#
# Reference: ulacache/telemetry/sparse_trace.py:11-263 (SparseTraceGeometry, historical_lookup_reference,
# GpuSparseTraceRecorder with chunk drains, events and expiry observations),
# ulacache/csrc/telemetry/sparse_trace.cuh.

from dataclasses import dataclass


@dataclass(frozen=True)
class SparseTraceGeometry:
    groups: int
    query_rows: int
    topk: int
    frames: int = 512
    chunk_frames: int = 64
    event_capacity: int = 262144

    def __post_init__(self):
        for name in ("groups", "query_rows", "topk", "frames", "chunk_frames", "event_capacity"):
            v = getattr(self, name)
            if type(v) is not int or not 0 < v < 2 ** 31:
                raise ValueError(f"{name} must be a positive int32 count")
        if self.frames % self.chunk_frames:
            raise ValueError("the trace window holds whole chunks")

    @property
    def payload_bytes(self) -> int:
        slots = self.chunk_frames * self.groups
        return (slots * self.query_rows * (self.topk + 1) * 4      # selections and current records
                + slots * (4 + 8)                                   # rows seen, epoch
                + self.event_capacity * 3 * 8 + 5 * 8)              # events, control


def historical_lookups(selected, query_requests, current):
    """The lookups one frame really makes, as a set of (request, id): padding (ids <= 0) and rows without a request
    are dropped, an id that ANY row of the same request is writing in this frame is not a lookup (it is resident by
    construction), and the same id asked for by several rows of one request counts once.  Equal ids of different
    requests stay distinct.  A CPU oracle for tests and trace conversion, not a scheduler."""
    if len(selected) != len(query_requests) or len(current) != len(query_requests):
        raise ValueError("one selection row, one request and one current record per query")
    written = {}
    for request, uid in zip(query_requests, current):
        if request >= 0 and uid >= 0:
            written.setdefault(int(request), set()).add(int(uid))
    out = set()
    for request, row in zip(query_requests, selected):
        if request < 0:
            continue
        mine = written.get(int(request), ())
        out.update((int(request), int(uid)) for uid in row if uid > 0 and int(uid) not in mine)
    return frozenset(out)


EVENT_ALLOCATE, EVENT_RELEASE = 1, 2
_ERR_BOUNDS, _ERR_EVENTS = 1, 2


class FramedSparseTrace:
    """control = (armed, frame, valid rows, error bits, events written) as int64 on the device."""

    def __init__(self, geometry: SparseTraceGeometry, *, device, max_gpu_bytes: int = 3_000_000_000):
        import torch

        if not isinstance(geometry, SparseTraceGeometry):
            raise TypeError("pass a SparseTraceGeometry")
        if type(max_gpu_bytes) is not int or geometry.payload_bytes > max_gpu_bytes:
            raise ValueError("the trace buffers exceed the diagnostic allowance")
        g = self.geometry = geometry
        slots = g.chunk_frames * g.groups
        i32, i64 = dict(dtype=torch.int32, device=device), dict(dtype=torch.int64, device=device)
        self.control = torch.zeros(5, **i64)
        # one spare slot at the end takes the writes of a disarmed or out-of-window observer
        self.selected = torch.zeros((slots + 1, g.query_rows, g.topk), **i32)
        self.current = torch.zeros((slots + 1, g.query_rows), **i32)
        self.seen = torch.full((slots + 1,), -1, **i32)
        self.epochs = torch.zeros((slots + 1,), **i64)
        self.events = torch.zeros((g.event_capacity + 1, 3), **i64)
        self._next_frame = self._drained = 0
        self._valid_rows = []

    @property
    def gpu_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in
                   (self.control, self.selected, self.current, self.seen, self.epochs, self.events))

    def start(self):
        """Arm at a quiescent boundary (after the state the replay starts from has been saved)."""
        self.control.zero_()
        self.control[0] = 1
        self.seen.fill_(-1)
        self._next_frame = self._drained = 0
        self._valid_rows = []

    def stop(self):
        self.control[0] = 0

    def begin_frame(self, valid_query_rows: int):
        """Outside the model's graph; nothing is read back."""
        g = self.geometry
        if type(valid_query_rows) is not int or not 0 <= valid_query_rows <= g.query_rows:
            raise ValueError("more valid query rows than the capture was sized for")
        if self._next_frame >= g.frames:
            raise ValueError("the declared trace window is full")
        if self._next_frame - self._drained >= g.chunk_frames:
            raise RuntimeError("drain the completed chunk before it is overwritten")
        self.control[1] = self._next_frame
        self.control[2] = valid_query_rows
        self._valid_rows.append(valid_query_rows)
        self._next_frame += 1

    def _slot(self, group: int):
        """Device scalar: the (frame, group) slot, or the spare slot when disarmed / outside the window."""
        import torch

        g = self.geometry
        armed, frame = self.control[0], self.control[1]
        ok = (armed > 0) & (frame >= 0) & (frame < g.frames)
        slot = (frame % g.chunk_frames) * g.groups + group
        return torch.where(ok, slot, torch.full_like(slot, g.chunk_frames * g.groups)).reshape(1)

    def observe(self, group: int, indices, current, epoch):
        """``indices`` int32 [rows <= query_rows, width <= topk], ``current`` int32 [rows], ``epoch`` a device
        scalar or int.  Bind immediately before the residency transaction of the group's selection."""
        import torch

        g = self.geometry
        if type(group) is not int or not 0 <= group < g.groups:
            raise ValueError("invalid residency group")
        rows, width = indices.shape
        if rows > g.query_rows or width > g.topk or current.shape[0] != rows:
            raise ValueError("the observed selection is larger than the capture was sized for")
        slot = self._slot(group)
        sel = torch.zeros((1, g.query_rows, g.topk), dtype=torch.int32, device=indices.device)
        sel[0, :rows, :width] = indices
        cur = torch.full((1, g.query_rows), -1, dtype=torch.int32, device=indices.device)
        cur[0, :rows] = current
        self.selected.index_copy_(0, slot, sel)
        self.current.index_copy_(0, slot, cur)
        self.seen.index_copy_(0, slot, self.control[2].to(torch.int32).reshape(1))
        ep = epoch if torch.is_tensor(epoch) else torch.tensor(int(epoch), device=indices.device)
        self.epochs.index_copy_(0, slot, ep.to(torch.int64).reshape(1))

    def observe_event(self, rows, *, release: bool):
        """Log allocation (``release=False``) or release of the records ``rows`` at the current frame."""
        import torch

        if type(release) is not bool:
            raise ValueError("say whether the event allocates or releases")
        g = self.geometry
        rows = rows.reshape(-1).to(torch.int64)
        n = rows.numel()
        if n == 0:
            return
        at = self.control[4]
        armed = self.control[0] > 0
        fits = at + n <= g.event_capacity
        dest = torch.where(armed & fits, at + torch.arange(n, device=rows.device),
                           torch.full((n,), g.event_capacity, dtype=torch.int64, device=rows.device))
        payload = torch.stack([self.control[1].expand(n), torch.full_like(rows, EVENT_RELEASE if release else EVENT_ALLOCATE),
                               rows], dim=1)
        self.events.index_copy_(0, dest, payload)
        self.control[4] += torch.where(armed & fits, n, 0)
        self.control[3] |= torch.where(armed & ~fits, _ERR_EVENTS, 0)

    def drain_chunk(self) -> dict:
        """A synchronising boundary: one complete chunk of frames comes to the host; every group must have been
        observed in every frame with the frame's row count."""
        import torch

        g = self.geometry
        count = self._next_frame - self._drained
        if count != g.chunk_frames:
            raise RuntimeError("only a complete chunk can be drained")
        if self.control.is_cuda:
            torch.cuda.synchronize(self.control.device)
        status = self.control.cpu().tolist()
        if status[3]:
            raise RuntimeError(f"the sparse trace recorded error bits {status[3]}")
        slots = g.chunk_frames * g.groups
        shape = (g.chunk_frames, g.groups)
        out = dict(first_frame=self._drained, frame_count=count,
                   selected=self.selected[:slots].cpu().reshape(*shape, g.query_rows, g.topk),
                   current=self.current[:slots].cpu().reshape(*shape, g.query_rows),
                   seen=self.seen[:slots].cpu().reshape(shape), epochs=self.epochs[:slots].cpu().reshape(shape))
        want = torch.tensor(self._valid_rows[self._drained:self._next_frame], dtype=torch.int32)[:, None].expand(shape)
        if not torch.equal(out["seen"], want):
            raise RuntimeError("a frame misses a residency group or disagrees on its query rows")
        self._drained = self._next_frame
        self.seen.fill_(-1)
        return out

    def event_snapshot(self):
        import torch

        if self.control.is_cuda:
            torch.cuda.synchronize(self.control.device)
        status = self.control.cpu().tolist()
        if status[3] & _ERR_EVENTS or not 0 <= status[4] <= self.geometry.event_capacity:
            raise RuntimeError("the event log overflowed")
        return self.events[:status[4]].cpu()


def frames_to_lookups(chunk: dict, query_requests, group: int = 0):
    """Per frame of a drained chunk: (sorted ids, their requests) of the lookups of one residency group, in the
    form the policy replays take.  ``query_requests``: request of every query row (-1 = none)."""
    out = []
    for f in range(chunk["frame_count"]):
        rows = int(chunk["seen"][f, group])
        pairs = sorted(historical_lookups(chunk["selected"][f, group, :rows].tolist(), list(query_requests[:rows]),
                                          chunk["current"][f, group, :rows].tolist()))
        out.append(([uid for _, uid in pairs], [req for req, _ in pairs]))
    return out
