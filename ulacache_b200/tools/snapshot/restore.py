"""Restore a request of ANY snapshot topology into this cache: the owners' stripes are read side by side and
re-interleaved into sequence order chunk by chunk, and the records' placements are resolved once per request
instead of once per layer.

``iter_sequence_plane`` consumes one byte stream per owner (position ``p`` of the request is row ``p // owners`` of
owner ``p % owners``) and yields (first position, uint8 [rows, width]) in sequence order with bounded memory; every
stream must end exactly where the request's geometry says.  ``PreparedSequenceRestore`` looks the target ids up in
each residency group's directory ONCE (device slot or host slot per record) and then writes any layer's chunk with
two index copies, one per tier: a 61-layer restore does one directory lookup, not 61.  The records must be
allocated and must not move while the restore runs, so it holds the cache quiescent.

Reference: ulacache/tools/snapshot/restore.py:8-349 (iter_sequence_plane, write_sequence_records,
PreparedSequenceRestore, restore_public_request).
"""
from __future__ import annotations

from typing import Iterator, Tuple


def iter_sequence_plane(reader, request_key: str, plane: str, *, chunk_rows: int = 8192) -> Iterator[Tuple[int, object]]:
    import torch

    owners = reader.layout.owners
    if type(chunk_rows) is not int or chunk_rows < owners or chunk_rows % owners:
        raise ValueError("a sequence chunk holds whole owner stripes")
    request = next((r for r in reader.requests if r.key == request_key), None)
    if request is None:
        raise ValueError("the snapshot holds no such request")
    width = reader.layout.planes()[plane]
    per_owner = chunk_rows // owners
    streams = [iter(reader.iter_plane(o, request_key, plane, chunk_bytes=per_owner * width)) for o in range(owners)]
    total = request.next_position
    for first in range(0, total, chunk_rows):
        count = min(chunk_rows, total - first)
        out = torch.empty((count, width), dtype=torch.uint8)
        for owner, stream in enumerate(streams):
            want = len(range(owner, count, owners))
            if not want:
                continue
            raw = next(stream, None)
            if raw is None or len(raw) != want * width:
                raise ValueError(f"owner {owner} of {plane} holds fewer records than the request's geometry")
            out[owner::owners] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(want, width)
        yield first, out
    for owner, stream in enumerate(streams):
        if next(stream, None) is not None:           # also runs the stream's size / hash check at its end
            raise ValueError(f"owner {owner} of {plane} holds more records than the request's geometry")


class PreparedSequenceRestore:
    """``ids``: the request's allocated logical ids in sequence order (this rank must own all of them)."""

    def __init__(self, cache, ids):
        import torch

        from ...transfer.file_io import QuiescentRecordIO

        self.cache, self.engine = cache, cache.engine
        if getattr(self.engine.owners, "ranks", 1) != 1:
            raise NotImplementedError("a striped pool restores per owner through cache_io.restore")
        self._guard = QuiescentRecordIO(cache)
        self._guard.__enter__()
        self.count = int(ids.numel())
        self.row_bytes = self.engine.storages[0].plane.bytes_per_record
        self._placements = []
        try:
            for res in self.engine.residency:
                flat = ids.reshape(-1).to(device=res.directory.device, dtype=torch.int32)
                mine, local = res._owned_locals(flat)
                if not bool(mine.all()):
                    raise ValueError("the restore targets ids this rank does not own")
                entry = res.directory[local.long()].cpu()
                if bool((entry == -1).any()):
                    raise ValueError("the restore targets ids without storage: allocate them first")
                dev_pos, host_pos = (entry >= 0).nonzero().flatten(), (entry <= -2).nonzero().flatten()
                self._placements.append((dev_pos, entry[dev_pos].long(), host_pos, (-entry[host_pos] - 2).long()))
        except BaseException:
            self._guard.__exit__(None, None, None)
            raise
        self.records_written = 0
        self.closed = False

    def write(self, layer: int, first: int, data, *, verify: bool = False):
        """``data`` uint8 [rows, record_bytes]: the records of sequence positions ``first ...`` of ``layer``."""
        import torch

        if self.closed:
            raise RuntimeError("the prepared restore is closed")
        if data.dtype != torch.uint8 or data.ndim != 2 or data.shape[1] != self.row_bytes:
            raise ValueError("snapshot chunks are whole records")
        rows = data.shape[0]
        if first < 0 or first + rows > self.count:
            raise ValueError("the chunk leaves the prepared request")
        eng = self.engine
        dev_pos, dev_slot, host_pos, host_slot = self._placements[eng.groups.group(layer)]
        for pos, slot, plane in ((dev_pos, dev_slot, eng.layer_plane(layer)), (host_pos, host_slot, eng.layer_host_plane(layer))):
            pick = ((pos >= first) & (pos < first + rows)).nonzero().flatten()
            if not pick.numel():
                continue
            if plane is None:
                raise RuntimeError("a record is placed in a host tier this cache does not have")
            src = data.index_select(0, pos[pick] - first)
            plane.index_copy_(0, slot[pick].to(plane.device), src.to(plane.device))
            if verify and not torch.equal(plane.index_select(0, slot[pick].to(plane.device)).cpu(), src):
                raise RuntimeError("restored records differ from the snapshot's bytes")
        self.records_written += rows

    def close(self):
        if not self.closed:
            self.closed = True
            self._guard.__exit__(None, None, None)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def restore_request(cache, reader, request_key: str, ids, *, verify: bool = False, chunk_rows: int = 8192,
                    index_writer=None) -> dict:
    """Restore one request of ``reader`` (any owner count) into ``ids`` of a single-owner cache.  Index planes go to
    ``index_writer(layer, ids_of_chunk, uint8 [rows, 132])`` when given.  Nothing is published to a request table."""
    lay = reader.layout
    plane0 = cache.cache_specification.storage_layout.record_planes[0]
    if lay.kv_format != plane0.native_encoding or lay.mla_row_bytes != plane0.bytes_per_record:
        raise ValueError("the snapshot's KV format does not match the cache")
    request = next((r for r in reader.requests if r.key == request_key), None)
    if request is None or int(ids.numel()) != request.next_position:
        raise ValueError("fresh ids must cover exactly the saved history of a request of this snapshot")
    chunk = max(lay.owners, chunk_rows // lay.owners * lay.owners)
    restored = 0
    with PreparedSequenceRestore(cache, ids) as prepared:
        for layer in range(lay.layers):
            for first, data in iter_sequence_plane(reader, request_key, f"mla_{layer:03d}", chunk_rows=chunk):
                prepared.write(layer, first, data, verify=verify)
                restored += data.numel()
    if index_writer is not None:
        for layer in lay.index_anchors:
            for first, data in iter_sequence_plane(reader, request_key, f"index_{layer:03d}", chunk_rows=chunk):
                index_writer(layer, ids[first:first + data.shape[0]], data)
                restored += data.numel()
    return dict(request_key=request_key, restored_bytes=restored, next_position=request.next_position,
                next_token_id=request.next_token_id, source_owners=lay.owners)
