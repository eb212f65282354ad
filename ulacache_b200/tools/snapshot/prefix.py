"""Single-request prefix snapshots: save one request's history out of bound byte banks, restore it into freshly
allocated records, and convert a one-owner prefix into owner stripes off line.

A prefix snapshot has one owner and describes SEQUENCE POSITIONS, not slots: row ``p`` of a plane is token ``p``.
Who produces and who consumes the bytes is the caller's business; :class:`ByteBanks` is the adapter over this
framework's storage (a record plane ``[layers, slots, record_bytes]`` and the Index page pools of the anchor
layers), addressed by the rows the caller allocated.  Producers must have retired before a save and consumers
must not have been told about the rows before a restore returns: both take a ``quiesce`` callable for that.

``stripe_prefix`` turns such a snapshot into an ``owners``-striped one (owner ``o`` keeps positions ``o, o + owners,
...``) so that every rank of a pool can read its share directly.  It streams: at most ``chunk_rows`` rows of one
plane are in memory at a time, whatever the length of the history.

Reference: ulacache/tools/snapshot/prefix.py:19-236 (stripe_prefix, write_prefix, iter_prefix_records,
NativeByteBanks, save_native_prefix, restore_native_prefix).
"""
from __future__ import annotations

import os
from dataclasses import replace
from typing import Callable, Dict, Iterator, Sequence, Tuple

from .format import SnapshotLayout, SnapshotReader, SnapshotRequest, SnapshotWriter, finalize_snapshot


def write_prefix(path: str, layout: SnapshotLayout, request: SnapshotRequest, read_records: Callable,
                 *, chunk_rows: int = 4096) -> dict:
    """Save one complete request.  ``read_records(plane, first, count) -> bytes`` returns exactly ``count`` rows of
    the plane starting at sequence position ``first``."""
    if layout.owners != 1 or type(chunk_rows) is not int or chunk_rows < 1:
        raise ValueError("a prefix snapshot has one owner; chunks hold at least one row")
    writer = SnapshotWriter(path, layout, [request], 0)
    total = request.next_position
    for plane, width in layout.planes().items():

        def chunks(plane=plane, width=width):
            for first in range(0, total, chunk_rows):
                count = min(chunk_rows, total - first)
                raw = read_records(plane, first, count)
                if len(raw) != count * width:
                    raise ValueError(f"the reader returned {len(raw)} bytes for {count} rows of {plane}")
                yield raw

        writer.write_plane(request.key, plane, chunks())
    writer.finish()
    return finalize_snapshot(path)


def iter_prefix_records(path: str, key: str, plane: str, *, chunk_rows: int = 4096) -> Iterator[Tuple[int, bytes]]:
    """(first position, checked bytes) per chunk of one plane of a one-owner snapshot; the hash is verified when
    the iterator is exhausted."""
    reader = SnapshotReader(path)
    if reader.layout.owners != 1:
        raise ValueError("a striped snapshot is read per owner, not as one sequence")
    width = reader.layout.planes()[plane]
    position = 0
    for raw in reader.iter_plane(0, key, plane, chunk_bytes=chunk_rows * width):
        if len(raw) % width:
            raise ValueError("the plane ends inside a record")
        yield position, raw
        position += len(raw) // width


def stripe_prefix(source: str, destination: str, owners: int, *, chunk_rows: int = 65536) -> dict:
    """Off-line conversion of a checked one-owner, one-request prefix into ``owners`` stripes.  Every row is kept,
    an uneven last stripe included; nothing is recomputed or requantised.  ``chunk_rows`` bounds memory (it is
    rounded to a multiple of ``owners`` so that a chunk splits evenly)."""
    import numpy as np

    reader = SnapshotReader(source, verify_payload=True)
    if reader.layout.owners != 1 or len(reader.requests) != 1:
        raise ValueError("stripe one request of a one-owner snapshot at a time")
    if type(owners) is not int or owners < 1 or type(chunk_rows) is not int or chunk_rows < 1:
        raise ValueError("owners and chunk rows are positive integers")
    request = reader.requests[0]
    os.makedirs(destination, exist_ok=False)
    layout = replace(reader.layout, owners=owners)
    writers = [SnapshotWriter(destination, layout, [request], owner) for owner in range(owners)]
    step = max(owners, chunk_rows // owners * owners)
    for plane, width in layout.planes().items():

        def stripe(owner, plane=plane, width=width):
            # a multiple of ``owners`` rows per chunk: position p of a chunk belongs to owner p % owners
            for _, raw in iter_prefix_records(source, request.key, plane, chunk_rows=step):
                rows = np.frombuffer(raw, dtype=np.uint8).reshape(-1, width)
                part = rows[owner::owners]
                if part.shape[0]:
                    yield part.tobytes()

        for owner, writer in enumerate(writers):
            writer.write_plane(request.key, plane, stripe(owner))
    for writer in writers:
        writer.finish()
    return finalize_snapshot(destination)


class ByteBanks:
    """``records``: uint8 [layers, slots, record_bytes] (any device); ``index``: {anchor layer: uint8 [pages,
    page bytes]} with segment-major pages (all keys of the page's rows, then all scales)."""

    def __init__(self, records, index: Dict[int, object] = None, *, index_segments: Sequence[int] = (128, 4),
                 page_rows: int = 64, kv_format: str = "mla.scaled656.fp8.v1"):
        import torch

        if records.ndim != 3 or records.dtype != torch.uint8:
            raise ValueError("records are uint8 [layers, slots, record_bytes]")
        self.records = records
        self.index = dict(index or {})
        self.row_bytes = int(records.shape[2])
        self.index_segments = tuple(int(w) for w in index_segments)
        self.page_rows, self.kv_format = int(page_rows), kv_format
        want = self.page_rows * sum(self.index_segments)
        for layer, pool in self.index.items():
            if not 0 <= layer < records.shape[0] or pool.ndim != 2 or pool.dtype != torch.uint8 or pool.shape[1] < want:
                raise ValueError("an Index pool is uint8 [pages, >= page_rows * row bytes] of a layer of the bank")

    @property
    def layers(self) -> int:
        return int(self.records.shape[0])

    def layout(self, fingerprint: str) -> SnapshotLayout:
        return SnapshotLayout(model_fingerprint=fingerprint, owners=1, layers=self.layers, mla_row_bytes=self.row_bytes,
                              index_anchors=tuple(sorted(self.index)), index_segment_bytes=self.index_segments,
                              index_page_rows=self.page_rows, kv_format=self.kv_format)

    @staticmethod
    def _layer(plane: str) -> int:
        return int(plane.rsplit("_", 1)[1])

    def read(self, plane: str, rows) -> bytes:
        import torch

        from .cache_io import read_index_records

        layer = self._layer(plane)
        if plane.startswith("mla_"):
            bank = self.records[layer]
            out = bank.index_select(0, rows.to(device=bank.device, dtype=torch.int64))
        else:
            pool = self.index[layer]
            out = read_index_records(pool, rows.to(pool.device), page_tokens=self.page_rows,
                                     segment_bytes=self.index_segments)
        return out.cpu().contiguous().numpy().tobytes()

    def write(self, plane: str, rows, raw: bytes, *, verify: bool = False):
        import torch

        from .cache_io import write_index_records

        layer = self._layer(plane)
        width = self.row_bytes if plane.startswith("mla_") else sum(self.index_segments)
        data = torch.frombuffer(bytearray(raw), dtype=torch.uint8).reshape(-1, width)
        if int(rows.numel()) != data.shape[0]:
            raise ValueError("the allocated rows do not cover the records of the chunk")
        if plane.startswith("mla_"):
            bank = self.records[layer]
            bank.index_copy_(0, rows.to(device=bank.device, dtype=torch.int64), data.to(bank.device))
        else:
            write_index_records(self.index[layer], rows, data, page_tokens=self.page_rows,
                                segment_bytes=self.index_segments)
        if verify and self.read(plane, rows) != raw:
            raise RuntimeError(f"restored bytes of {plane} differ from the snapshot")


def save_prefix_from_banks(path: str, request: SnapshotRequest, banks: ByteBanks, rows, fingerprint: str,
                           *, quiesce: Callable[[], None]) -> dict:
    """``rows[p]`` is the bank row of sequence position ``p``.  ``quiesce`` returns once every producer of those
    rows has retired."""
    if int(rows.numel()) != request.next_position:
        raise ValueError("the rows must cover exactly the saved history")
    quiesce()
    return write_prefix(path, banks.layout(fingerprint), request,
                        lambda plane, first, count: banks.read(plane, rows[first:first + count]))


def restore_prefix_to_banks(path: str, key: str, banks: ByteBanks, rows, fingerprint: str, *,
                            quiesce: Callable[[], None], verify: bool = False, chunk_rows: int = 4096) -> dict:
    """Write the request's records into rows the caller allocated and has not published yet.  The snapshot must
    have been taken from banks of the same geometry and fingerprint."""
    reader = SnapshotReader(path)
    lay = reader.layout
    if lay != banks.layout(fingerprint):
        raise ValueError("the snapshot and the bound banks differ in geometry, format or fingerprint")
    request = next((r for r in reader.requests if r.key == key), None)
    if request is None or int(rows.numel()) != request.next_position:
        raise ValueError("fresh rows must cover exactly the saved history of a request of this snapshot")
    quiesce()
    restored = 0
    for plane in lay.planes():
        at = 0
        for first, raw in iter_prefix_records(path, key, plane, chunk_rows=chunk_rows):
            count = len(raw) // lay.planes()[plane]
            banks.write(plane, rows[first:first + count], raw, verify=verify)
            at = first + count
            restored += len(raw)
        if at != request.next_position:
            raise ValueError(f"{plane} does not cover the saved history")
    quiesce()
    return dict(request_key=key, restored_bytes=restored, next_position=request.next_position,
                next_token_id=request.next_token_id)
