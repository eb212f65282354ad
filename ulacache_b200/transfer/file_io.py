"""File-backed record sources: restore KV records from a snapshot plane into the
cache through its normal directory routing.

A ``FileRecordSource`` names complete native records inside a file (local disk or a parallel file system):
a byte range, or every ``record_stride``-th record of one (an owner's stripe of a whole-request plane).  It
can bind the file's size and the SHA-256 of the selected records in order.  ``FileRecordReader`` reads it
into buffers the caller owns (``readinto`` hands out a lease on the buffer; the last chunk is handed out only
after size, end-of-file and hash checks passed) or iterates it in bounded chunks.  ``restore_file_records``
streams a source through two pinned buffers, so that the file read of one chunk runs under the host-to-device
copy and the routed write of the previous one.

Reference: ulacache/transfer/file_io.py (FileRecordSource :17, PlaneChunk :182, FileRecordReader
:203, NativeRecordRouting :390, QuiescentRecordIO :549).
"""
from __future__ import annotations

import hashlib
import mmap
import os
import time
from dataclasses import dataclass, replace
from typing import Optional

DEFAULT_CHUNK_BYTES = 64 << 20
_HEX = set("0123456789abcdef")


@dataclass(frozen=True)
class FileRecordSource:
    path: str
    offset: int
    record_count: int
    row_bytes: int
    native_encoding: str
    sha256: str = ""                     # of the selected records, in order (headers and gaps excluded)
    file_bytes: Optional[int] = None     # exact size of the file; None: it only has to cover the range
    record_stride: int = 1               # every stride-th record starting at ``offset``
    verify_payload: Optional[bool] = None    # None: verify exactly when a hash is given

    def __post_init__(self):
        ints = (self.offset, self.record_count, self.row_bytes, self.record_stride)
        if any(type(v) is not int for v in ints):
            raise ValueError("Offset, record count, row bytes and stride are integers")
        if self.offset < 0 or self.record_count < 0 or self.row_bytes <= 0 or self.record_stride < 1:
            raise ValueError("Invalid file record range")
        digest = self.sha256.lower()
        if digest and (len(digest) != 64 or set(digest) - _HEX):
            raise ValueError("The payload hash is 64 hexadecimal digits")
        object.__setattr__(self, "sha256", digest)
        verify = bool(digest) if self.verify_payload is None else self.verify_payload
        if type(verify) is not bool:
            raise ValueError("verify_payload is a boolean")
        if verify and not digest:
            raise ValueError("Verification needs the hash of the selected records")
        object.__setattr__(self, "verify_payload", verify)
        if self.file_bytes is not None and (type(self.file_bytes) is not int or self.file_bytes < self.range_end):
            raise ValueError("The declared file size does not cover the selected records")

    @property
    def nbytes(self) -> int:
        return self.record_count * self.row_bytes

    @property
    def range_end(self) -> int:
        """One past the last selected byte of the file."""
        if self.record_count == 0:
            return self.offset
        return self.offset + ((self.record_count - 1) * self.record_stride + 1) * self.row_bytes

    def slice(self, first: int, count: int) -> "FileRecordSource":
        """Records ``[first, first + count)`` of this source.  The whole-range hash says nothing about a part,
        so the slice carries none."""
        if first < 0 or count < 0 or first + count > self.record_count:
            raise ValueError("Slice outside the source")
        return replace(self, offset=self.offset + first * self.record_stride * self.row_bytes, record_count=count,
                       sha256="", verify_payload=False)

    def select_owner(self, owner: int, owners: int) -> "FileRecordSource":
        """The records ``owner, owner + owners, ...`` of this source (a position stripe).  A source that must be
        verified cannot be striped: its hash covers all records; verify it whole first, or use a snapshot that was
        written per owner."""
        if type(owners) is not int or owners < 1 or type(owner) is not int or not 0 <= owner < owners:
            raise ValueError("Name a valid owner of the stripe")
        if self.verify_payload:
            raise ValueError("A stripe of a hashed source cannot be verified; verify the whole source first")
        count = len(range(owner, self.record_count, owners))
        offset = self.offset + owner * self.record_stride * self.row_bytes
        if count == 0:
            offset = min(offset, self.range_end)
        return replace(self, offset=offset, record_count=count, record_stride=self.record_stride * owners, sha256="")

    @classmethod
    def from_snapshot(cls, reader, request_key: str, plane: str, *, owner=None, verify_payload=None):
        """One owner's file of one request and plane of a committed snapshot, bound to the size and hash that the
        owner's receipt records.  ``reader``: :class:`~ulacache_b200.tools.snapshot.format.SnapshotReader`."""
        owners = reader.layout.owners
        if owner is None:
            if owners != 1:
                raise ValueError("A snapshot with several owners needs the owner named")
            owner = 0
        receipt = reader.validate_owner(owner)
        path = reader.plane_file(owner, request_key, plane)
        rec = receipt["files"][os.path.basename(path)]
        width = reader.layout.planes()[plane]
        rows = reader.plane_rows(owner, request_key)
        if rec["bytes"] != rows * width:
            raise ValueError("The plane file does not match its request's geometry")
        verify = reader.verify_payload if verify_payload is None else bool(verify_payload)
        encoding = reader.layout.kv_format if plane.startswith("mla_") else plane.split("_")[0]
        return cls(path, 0, rows, width, encoding, sha256=rec["sha256"] if verify else "", file_bytes=rec["bytes"],
                   verify_payload=verify)

    def open(self, chunk_bytes: int = DEFAULT_CHUNK_BYTES) -> "FileRecordReader":
        return FileRecordReader(self, chunk_bytes)


class LeasedChunk:
    """Records ``[first, first + data.shape[0])`` of the source in the caller's buffer.  The buffer stays leased
    until :meth:`release`; ``release(after=event.synchronize)`` waits for a consumer first and keeps the lease when
    the wait raises."""

    def __init__(self, reader, token, first, data):
        self.first, self.data = first, data
        self._reader, self._token = reader, token
        self.released = False

    def release(self, *, after=None):
        if self.released:
            return
        if after is not None:
            after()
        self._reader._leases.pop(self._token, None)
        self.released = True


class FileRecordReader:
    """Bounded, read-only access to a source.  Closing the reader closes the file; leased buffers stay the caller's."""

    def __init__(self, source: FileRecordSource, chunk_bytes: int = DEFAULT_CHUNK_BYTES):
        if chunk_bytes < source.row_bytes:
            raise ValueError("A chunk must hold at least one record")
        self.source = source
        self.rows_per_chunk = max(1, chunk_bytes // source.row_bytes)
        self._t0 = time.perf_counter()
        self._digest = hashlib.sha256() if source.verify_payload else None
        self._leases = {}
        self._next_token = 0
        self._rows_read = 0
        self._verified = False
        self._closed = False
        self._map = None
        self.bytes_read = self.chunks_read = 0
        self.wall_seconds = None
        self._fd = os.open(source.path, os.O_RDONLY)
        try:
            self._check_size()
            if source.record_stride > 1 and source.record_count:
                self._map = mmap.mmap(self._fd, 0, access=mmap.ACCESS_READ)
        except BaseException:
            self.close()
            raise

    def _check_size(self):
        size, s = os.fstat(self._fd).st_size, self.source
        if s.file_bytes is not None and size != s.file_bytes:
            raise ValueError(f"{s.path} is truncated or extended: {size} bytes, {s.file_bytes} declared")
        if size < s.range_end:
            raise ValueError(f"{s.path} is shorter than the declared record range")

    # --------------------------------------------------------------- leased reads --
    def readinto(self, buffer) -> Optional[LeasedChunk]:
        """Fill ``buffer`` (contiguous CPU uint8 [rows, row_bytes], pinned or not) with the next records.  Returns
        None after the verified end.  A buffer that overlaps a live lease is refused."""
        import numpy as np
        import torch

        if self._closed:
            raise RuntimeError("The file reader is closed")
        s = self.source
        if self._verified:
            return None
        if self._rows_read == s.record_count:
            self._finish()
            return None
        if (not isinstance(buffer, torch.Tensor) or buffer.device.type != "cpu" or buffer.dtype != torch.uint8
                or buffer.ndim != 2 or buffer.shape[1] != s.row_bytes or buffer.shape[0] < 1 or not buffer.is_contiguous()):
            raise ValueError("Supply a contiguous CPU uint8 [rows, row_bytes] buffer")
        lo, hi = buffer.data_ptr(), buffer.data_ptr() + buffer.numel()
        if any(lo < b and a < hi for a, b in self._leases.values()):
            raise RuntimeError("A consumer still holds a lease on this buffer")
        first = self._rows_read
        n = min(buffer.shape[0], s.record_count - first)
        out = buffer[:n]
        try:
            if self._map is not None:
                self._check_size()
                whole = np.frombuffer(self._map, dtype=np.uint8)
                start = s.offset + first * s.record_stride * s.row_bytes
                picked = np.lib.stride_tricks.as_strided(whole[start:], (n, s.row_bytes), (s.record_stride * s.row_bytes, 1),
                                                         writeable=False)
                out.numpy()[...] = picked
                del picked, whole
            else:
                view = memoryview(out.numpy()).cast("B")
                at, end = s.offset + first * s.row_bytes, n * s.row_bytes
                done = 0
                while done < end:
                    got = os.preadv(self._fd, [view[done:]], at + done)
                    if got <= 0:
                        raise ValueError(f"{s.path} ended inside its declared records")
                    done += got
            if self._digest is not None:
                self._digest.update(memoryview(out.numpy()).cast("B"))
        except BaseException:
            self.close()
            raise
        self._rows_read += n
        self.bytes_read += n * s.row_bytes
        self.chunks_read += 1
        if self._rows_read == s.record_count:
            self._finish()                      # the last chunk leaves only after the whole range checked out
        token = self._next_token
        self._next_token += 1
        self._leases[token] = (lo, hi)
        return LeasedChunk(self, token, first, out)

    def _finish(self):
        try:
            self._check_size()
            if self._digest is not None and self._digest.hexdigest() != self.source.sha256:
                raise ValueError(f"{self.source.path}: payload checksum mismatch")
        except BaseException:
            self.close()
            raise
        self._verified = True

    # ------------------------------------------------------------------ iteration --
    def __iter__(self):
        """(first record, fresh uint8 [n, row_bytes] tensor) per chunk; the last one only after verification."""
        import torch

        while True:
            left = self.source.record_count - self._rows_read
            if left <= 0 and self._verified:
                return
            buf = torch.empty((max(1, min(self.rows_per_chunk, left)), self.source.row_bytes), dtype=torch.uint8)
            chunk = self.readinto(buf)
            if chunk is None:
                return
            chunk.release()
            yield chunk.first, chunk.data

    def statistics(self) -> dict:
        return dict(bytes_read=self.bytes_read, chunks_read=self.chunks_read, end_verified=self._verified,
                    payload_sha256_verified=bool(self._digest is not None and self._verified),
                    leased_buffers=len(self._leases), closed=self._closed, wall_seconds=self.wall_seconds)

    def close(self):
        if self._closed:
            return
        if self._map is not None:
            self._map.close()
            self._map = None
        os.close(self._fd)
        self._closed = True
        self.wall_seconds = time.perf_counter() - self._t0

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def restore_file_records(engine, layer: int, ids, source: FileRecordSource,
                         chunk_bytes: int = DEFAULT_CHUNK_BYTES, statistics=None) -> int:
    """Blocking restore: stream the source and publish each chunk through the engine's writer, which routes by
    directory.  On a GPU the chunks alternate between two pinned buffers: chunk ``i + 1`` is read from the file while
    chunk ``i`` is copied and written on the stream; a buffer is reused only after the event recorded behind its write
    has completed.  Returns the number of records written.  A hash mismatch raises after the records before the last
    chunk were written: the caller frees the ids (nothing has been published to a request table)."""
    import torch

    flat = ids.reshape(-1)
    cuda = engine.device.type == "cuda"
    rows = max(1, min(chunk_bytes // source.row_bytes, max(1, source.record_count)))
    buffers = [torch.empty((rows, source.row_bytes), dtype=torch.uint8) for _ in range(2 if cuda else 1)]
    if cuda:
        buffers = [b.pin_memory() for b in buffers]
    pending = [None] * len(buffers)
    done = turn = 0
    with FileRecordReader(source, chunk_bytes) as reader:
        try:
            while True:
                slot = turn % len(buffers)
                if pending[slot] is not None:
                    chunk, event = pending[slot]
                    chunk.release(after=event.synchronize if event is not None else None)
                    pending[slot] = None
                chunk = reader.readinto(buffers[slot])
                if chunk is None:
                    break
                n = chunk.data.shape[0]
                payload = chunk.data.to(engine.device, non_blocking=True) if cuda else chunk.data
                engine.write(layer, flat[chunk.first:chunk.first + n], payload)
                event = None
                if cuda:
                    event = torch.cuda.Event()
                    event.record()
                pending[slot] = (chunk, event)
                done += n
                turn += 1
        finally:
            for item in pending:
                if item is not None:
                    item[0].release(after=item[1].synchronize if item[1] is not None else None)
        if statistics is not None:
            statistics.update(reader.statistics())
    return done


class QuiescentRecordIO:
    """Guard for snapshot save / restore: refuses to run while a forward holds views."""

    def __init__(self, cache):
        self.cache = cache

    def __enter__(self):
        self.cache._access.require_idle("snapshot I/O")
        if self.cache.engine.device.type == "cuda":
            import torch

            torch.cuda.synchronize(self.cache.engine.device)
        return self

    def __exit__(self, *exc):
        if self.cache.engine is not None and self.cache.engine.device.type == "cuda":
            import torch

            torch.cuda.synchronize(self.cache.engine.device)
        return False
