"""Receive side of prefill/decode disaggregation: a remote prefill worker writes KV records
straight into this rank's canonical record storage, so the plan is a list of byte extents.

    plan = plan_direct_receive(slots, record_bytes=656, layers=61, layer_stride=..., base_address=...)
    # -> per layer: coalesced (address, bytes) extents the sender's RDMA writes target
    window = OrderedReceiveWindow(chunks=plan.chunk_count)
    window.accept(seq) ...                       # completions may arrive out of order
    publish_received(engine, ids, window)        # ids become visible only when every chunk landed

Records whose destination is the host tier are planned against the pinned host plane the same way
(``tier="host"``).  No transport is implemented here: the extents are what a transport (RDMA, or a
peer copy in tests) consumes.

Reference: ulacache/transfer/direct_receive.py:528 (plans), direct_receiver.py, receive_window.py,
native_paged_receive.py, owner_receive_window.py, transfer/kernels/receive_publication.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple


@dataclass(frozen=True)
class Extent:
    address: int
    nbytes: int
    first_record: int       # index into the request's record list of the first record of the extent
    records: int


@dataclass(frozen=True)
class DirectReceivePlan:
    tier: str                                   # "device" | "host"
    record_bytes: int
    layers: int
    extents: Tuple[Tuple[Extent, ...], ...]     # per layer
    chunk_records: int

    @property
    def chunk_count(self) -> int:
        return sum(len(layer) for layer in self.extents)

    @property
    def total_bytes(self) -> int:
        return sum(e.nbytes for layer in self.extents for e in layer)


def coalesce_slots(slots: Sequence[int], max_records: int = 0) -> List[Tuple[int, int, int]]:
    """Runs of consecutive slots: (first position in ``slots``, first slot, run length), each run at
    most ``max_records`` long when that is positive."""
    runs = []
    i, n = 0, len(slots)
    while i < n:
        j = i + 1
        while j < n and slots[j] == slots[j - 1] + 1 and (max_records <= 0 or j - i < max_records):
            j += 1
        runs.append((i, int(slots[i]), j - i))
        i = j
    return runs


def plan_direct_receive(slots: Sequence[int], *, record_bytes: int, layers: int, layer_stride: int, base_address: int,
                        tier: str = "device", pool_slots: int = 0, chunk_records: int = 4096) -> DirectReceivePlan:
    """``slots``: destination slot of every record of the request, in token order (all in one tier).
    ``base_address``: address of slot 0 of layer 0; ``layer_stride``: bytes between layers."""
    if tier not in ("device", "host"):
        raise ValueError("tier must be device or host")
    if record_bytes <= 0 or record_bytes % 16 or layers < 1:
        raise ValueError("record_bytes must be a positive multiple of 16 and layers >= 1")
    slots = [int(s) for s in slots]
    if any(s < 0 or (pool_slots and s >= pool_slots) for s in slots):
        raise ValueError("destination slot outside the pool")
    if len(set(slots)) != len(slots):
        raise ValueError("two records target the same slot")
    runs = coalesce_slots(slots, chunk_records)
    per_layer = []
    for layer in range(layers):
        base = base_address + layer * layer_stride
        per_layer.append(tuple(Extent(base + s * record_bytes, n * record_bytes, pos, n) for pos, s, n in runs))
    return DirectReceivePlan(tier, record_bytes, layers, tuple(per_layer), chunk_records)


class OrderedReceiveWindow:
    """Completion tracking of a plan's chunks.  ``ready_prefix`` is the number of leading chunks
    (in plan order) that have all arrived: consumers that stream may read that far."""

    def __init__(self, chunks: int):
        if chunks < 0:
            raise ValueError("chunks >= 0")
        self.chunks = chunks
        self._done = [False] * chunks
        self.ready_prefix = 0
        self.arrived = 0

    def accept(self, seq: int):
        if not 0 <= seq < self.chunks:
            raise IndexError(f"chunk {seq} is not part of the plan")
        if self._done[seq]:
            raise ValueError(f"chunk {seq} completed twice")
        self._done[seq] = True
        self.arrived += 1
        while self.ready_prefix < self.chunks and self._done[self.ready_prefix]:
            self.ready_prefix += 1

    @property
    def complete(self) -> bool:
        return self.arrived == self.chunks

    def missing(self) -> List[int]:
        return [i for i, d in enumerate(self._done) if not d]


class ReceiveNotComplete(RuntimeError):
    pass


def publish_received(register, ids, window: OrderedReceiveWindow):
    """Make received records visible: ``register(ids)`` binds the ids to the slots the plan wrote
    (for a cache client: ``SlotManager.register``).  Refuses while chunks are outstanding."""
    if not window.complete:
        raise ReceiveNotComplete(f"chunks {window.missing()[:8]} have not arrived")
    return register(ids)


# ----------------------------------------------------------------------------------- plan on the wire --
# The receiver sends its plan to the prefill worker once per request.  Every layer has the same runs of
# destination slots and differs only in its base address, so the message is a small JSON header (tier, sizes,
# one base address per layer) followed by the runs as little-endian int64 triples (first record, first slot,
# records).  Reference: ulacache/transfer/direct_receive.py:390-525 (binary plan metadata with run compression).

PLAN_MAGIC = b"ULCRXPL1"
_MAX_HEADER = 1 << 16


def encode_plan(plan: DirectReceivePlan) -> bytes:
    import json
    import struct

    first = plan.extents[0] if plan.extents else ()
    runs = [(e.first_record, (e.address - first[0].address) // plan.record_bytes, e.records) for e in first]
    # slots relative to the layer's first extent keep the triples small; the header carries the absolute base
    header = json.dumps(dict(version=1, tier=plan.tier, record_bytes=plan.record_bytes, layers=plan.layers,
                             chunk_records=plan.chunk_records, runs=len(runs),
                             bases=[layer[0].address if layer else 0 for layer in plan.extents]),
                        separators=(",", ":")).encode()
    body = b"".join(struct.pack("<qqq", *r) for r in runs)
    return PLAN_MAGIC + struct.pack("<I", len(header)) + header + body


def decode_plan(payload: bytes, *, record_limit: int) -> DirectReceivePlan:
    """Rebuild a plan from :func:`encode_plan` output.  Everything is checked before it is believed: sizes,
    that the runs tile ``[0, records)`` without gaps, that no two runs overlap in the destination, and that the
    request does not exceed ``record_limit`` records."""
    import json
    import struct

    if type(record_limit) is not int or record_limit < 0:
        raise ValueError("a record limit is required")
    if len(payload) < 12 or payload[:8] != PLAN_MAGIC:
        raise ValueError("not a receive plan")
    (size,) = struct.unpack_from("<I", payload, 8)
    if size > _MAX_HEADER or 12 + size > len(payload):
        raise ValueError("receive plan header is cut short or oversized")
    h = json.loads(payload[12:12 + size])
    if h.get("version") != 1 or h.get("tier") not in ("device", "host"):
        raise ValueError("unknown receive plan version or tier")
    rb, layers, runs_n, bases = h["record_bytes"], h["layers"], h["runs"], h["bases"]
    if (type(rb) is not int or rb <= 0 or rb % 16 or type(layers) is not int or layers < 1 or type(runs_n) is not int
            or runs_n < 0 or len(bases) != layers or any(type(b) is not int or b < 0 for b in bases)):
        raise ValueError("receive plan header fields are malformed")
    if len(payload) != 12 + size + 24 * runs_n:
        raise ValueError("receive plan body does not match its run count")
    runs = [struct.unpack_from("<qqq", payload, 12 + size + 24 * i) for i in range(runs_n)]
    expect, taken = 0, []
    for pos, slot, n in runs:
        if pos != expect or n <= 0:
            raise ValueError("receive plan runs leave a gap or overlap in the request")
        expect += n
        taken.append((slot, slot + n))
    if expect > record_limit:
        raise ValueError("receive plan names more records than the request may carry")
    taken.sort()
    if any(a_end > b_start for (_, a_end), (b_start, _) in zip(taken, taken[1:])):
        raise ValueError("two runs of a receive plan share destination records")
    extents = tuple(tuple(Extent(base + slot * rb, n * rb, pos, n) for pos, slot, n in runs) for base in bases)
    return DirectReceivePlan(h["tier"], rb, layers, extents, int(h.get("chunk_records", 0)))


def iter_segments(plan: DirectReceivePlan, source_bases: Sequence[int], *, source_rows=None, first_record: int = 0,
                  record_count=None, max_segments: int = 4096):
    """Sender side: bounded batches of (source address, destination address, bytes) triples that move records
    ``[first_record, first_record + record_count)`` of the request in every layer.  ``source_bases``: per layer,
    the address of the sender's record 0; ``source_rows`` (optional): the sender's row of every request record
    (a paged source), otherwise records are consecutive at the source.  A segment never spans a break at either
    end and bytes are never reordered."""
    if type(max_segments) is not int or max_segments < 1:
        raise ValueError("at least one segment per batch")
    if len(source_bases) != plan.layers:
        raise ValueError("one source base per planned layer")
    total = sum(e.records for e in plan.extents[0]) if plan.extents else 0
    count = total - first_record if record_count is None else record_count
    if first_record < 0 or count < 0 or first_record + count > total:
        raise ValueError("the chunk leaves the planned records")
    if source_rows is not None and len(source_rows) < first_record + count:
        raise ValueError("the source names fewer rows than the chunk")
    rb = plan.record_bytes
    batch = []
    for layer in range(plan.layers):
        for e in plan.extents[layer]:
            lo, hi = max(e.first_record, first_record), min(e.first_record + e.records, first_record + count)
            if lo >= hi:
                continue
            i = lo
            while i < hi:
                j = i + 1
                if source_rows is not None:
                    while j < hi and source_rows[j] == source_rows[j - 1] + 1:
                        j += 1
                else:
                    j = hi
                src_row = source_rows[i] if source_rows is not None else i
                batch.append((source_bases[layer] + int(src_row) * rb, e.address + (i - e.first_record) * rb,
                              (j - i) * rb))
                if len(batch) == max_segments:
                    yield batch
                    batch = []
                i = j
    if batch:
        yield batch


def send_chunk(write, plan, source_bases, *, source_rows=None, first_record: int = 0, record_count=None,
               record_limit=None, executors=(), max_inflight: int = 16, max_segments: int = 4096, audit=None) -> int:
    """Drive ``write(batch) -> status`` (0 = ok) over the batches of one chunk.  ``plan`` may be the encoded
    message.  With ``executors`` (thread pools), up to ``max_inflight`` batches are in flight; after a failure no
    new batch starts, but every batch already submitted is joined before returning: a failed write is no proof
    that its DMA stopped, so the caller still has to drain the transport before the destinations are reused."""
    import time
    from concurrent.futures import FIRST_COMPLETED, wait

    t0 = time.monotonic()
    if isinstance(plan, (bytes, bytearray, memoryview)):
        if record_limit is None:
            raise ValueError("decoding a plan needs the request's record limit")
        plan = decode_plan(bytes(plan), record_limit=record_limit)
    if type(max_inflight) is not int or max_inflight < 1:
        raise ValueError("at least one batch in flight")
    executors = tuple(executors)
    status, error, pending = 0, None, set()
    stats = dict(batches=0, segments=0, bytes=0, peak_inflight=0, peak_segments=0)

    def collect(done):
        nonlocal status, error
        for f in done:
            try:
                rc = f.result()
            except BaseException as exc:                       # joined, reported after the drain
                rc, error = -1, error or exc
            if rc != 0 and status == 0:
                status = rc

    try:
        for batch in iter_segments(plan, source_bases, source_rows=source_rows, first_record=first_record,
                                   record_count=record_count, max_segments=max_segments):
            if status != 0:
                break
            stats["batches"] += 1
            stats["segments"] += len(batch)
            stats["bytes"] += sum(b[2] for b in batch)
            stats["peak_segments"] = max(stats["peak_segments"], len(batch))
            if executors:
                while len(pending) >= max_inflight:
                    done, pending = wait(pending, return_when=FIRST_COMPLETED)
                    collect(done)
                if status != 0:
                    break
                pending.add(executors[stats["batches"] % len(executors)].submit(write, batch))
                stats["peak_inflight"] = max(stats["peak_inflight"], len(pending))
            else:
                rc = write(batch)
                if rc != 0:
                    status = rc
    except BaseException as exc:
        status, error = status or -1, error or exc
    finally:
        if pending:
            done, _ = wait(pending)
            collect(done)
    if audit is not None:
        audit(dict(stats, status=status, seconds=time.monotonic() - t0, first_record=first_record,
                   max_segments=max_segments, max_inflight=max_inflight))
    if error is not None:
        raise error
    return status
