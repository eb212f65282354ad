"""Save request KV from a live cache into a snapshot shard, and restore it.

Saving runs under :class:`~ulacache_b200.transfer.file_io.QuiescentRecordIO` (no forward may
hold views).  Each snapshot owner ``r`` saves the rows of positions ``p % owners == r``; the
records are read through the cache's own access path (promotion from the host tier, peer reads),
so the snapshot is independent of where records happened to live.  Restoring streams every
owner's files through ``UlaCache.write(ids, layer, FileRecordSource)``; the writer routes each
record by directory and, with owner-only routing, every rank keeps exactly the records it owns.

Reference: CudaRequestSnapshot (ulacache/tools/snapshot/cuda.py:53) and the restore path
ulacache/tools/snapshot/restore.py.
"""
from __future__ import annotations

from typing import Dict, Sequence

from ...transfer.file_io import FileRecordSource, QuiescentRecordIO
from .format import SnapshotLayout, SnapshotReader, SnapshotRequest, SnapshotWriter


def save_shard(cache, path: str, layout: SnapshotLayout, requests: Sequence[SnapshotRequest],
               request_ids: Dict[str, object], owner: int, *, chunk_rows: int = 2048, index_reader=None):
    """``request_ids[key]``: int32 tensor of the request's logical IDs in position order.
    ``index_reader(layer, ids) -> uint8 [n, 132]`` supplies index records when the layout has index planes."""
    import torch

    writer = SnapshotWriter(path, layout, requests, owner)
    a = cache.cache_specification.sparse_access
    width = a.maximum_selected_record_count
    with QuiescentRecordIO(cache):
        for layer in range(layout.layers):
            plane = f"mla_{layer:03d}"
            for req in requests:
                ids = request_ids[req.key][: req.next_position][owner::layout.owners]

                def chunks():
                    for s in range(0, ids.numel(), min(chunk_rows, width)):
                        part = ids[s:s + min(chunk_rows, width)].reshape(1, -1).to(torch.int32)
                        cache.begin_model_forward()
                        cache.access(part, layer)
                        rows = cache.gather_selected_records(layer)
                        cache.finish_layer_attention(layer)
                        cache.finish_model_forward()
                        yield rows.cpu().numpy().tobytes()

                writer.write_plane(req.key, plane, chunks())
        for layer in layout.index_anchors:
            plane = f"index_{layer:03d}"
            for req in requests:
                ids = request_ids[req.key][: req.next_position][owner::layout.owners]
                rows = index_reader(layer, ids) if index_reader is not None else None
                if rows is None:
                    raise ValueError("The layout declares index planes but no index_reader was given")
                writer.write_plane(req.key, plane, [rows.cpu().numpy().tobytes()])
    return writer.finish()


def release_unwritten_padding(cache, allocated_ids, history_length: int):
    """A restored request was given whole pages of ids; only its real history is bound to records.  The ids of the
    page tail are released again, so that ordinary decode registers each later token exactly once when it is
    written (a speculative caller, which reserves whole pages on purpose, does not call this).

    Reference: ulacache/tools/snapshot/cuda.py:12-27 (release_unwritten_padding)."""
    n = int(allocated_ids.numel())
    if not 0 < history_length <= n:
        raise ValueError("the real history must fit the allocation")
    tail = allocated_ids[history_length:]
    if tail.numel():
        cache.release_logical_records(tail)
    return int(tail.numel())


def restore(cache, path: str, request_ids: Dict[str, object], *, verify_payload=None, index_writer=None,
            verify_restored: bool = False) -> int:
    """Write snapshot records back into ``cache`` under the given logical IDs: every saved request, or only those
    named in ``request_ids`` (a subset restores part of a bank).  ``verify_restored``: read every restored chunk back
    through the cache and compare it with the file's bytes.  Returns records written (counting each (layer, token)
    once per reading rank).  Nothing is published to a request table or prefix tree here: the caller does that
    after every owner's restore has succeeded."""
    reader = SnapshotReader(path, verify_payload=verify_payload)
    saved = {r.key for r in reader.requests}
    if not request_ids or not set(request_ids) <= saved:
        raise ValueError("restore needs fresh ids for requests the snapshot holds")
    lay = reader.layout
    plane0 = cache.cache_specification.storage_layout.record_planes[0]
    if lay.kv_format != plane0.native_encoding or lay.mla_row_bytes != plane0.bytes_per_record:
        raise ValueError("The snapshot's KV format does not match the cache")
    done = 0
    with QuiescentRecordIO(cache):
        for owner in range(lay.owners):
            for req in reader.requests:
                if req.key not in request_ids:
                    continue
                ids = request_ids[req.key][: req.next_position][owner::lay.owners]
                if ids.numel() == 0:
                    continue
                rows = reader.plane_rows(owner, req.key)
                for layer in range(lay.layers):
                    plane = f"mla_{layer:03d}"
                    # bound to the receipt's size and hash: the file is read once, hashed while it streams, and a
                    # mismatch raises out of the write (the caller frees the ids; nothing was published)
                    src = FileRecordSource.from_snapshot(reader, req.key, plane, owner=owner)
                    if src.record_count != rows:
                        raise ValueError("snapshot plane and request geometry differ")
                    done += cache.write(ids, layer, src)
                    if verify_restored:
                        _verify_restored(cache, layer, ids, reader, owner, req.key, plane, lay.mla_row_bytes)
                for layer in lay.index_anchors:
                    if index_writer is None:
                        continue
                    plane = f"index_{layer:03d}"
                    data = b"".join(reader.iter_plane(owner, req.key, plane))
                    index_writer(layer, ids, data)
    return done


def _verify_restored(cache, layer, ids, reader, owner, key, plane, row_bytes):
    import torch

    at = 0
    for raw in reader.iter_plane(owner, key, plane, chunk_bytes=max(row_bytes, (4 << 20) // row_bytes * row_bytes)):
        want = torch.frombuffer(bytearray(raw), dtype=torch.uint8).reshape(-1, row_bytes)
        got = cache.engine.read_records(layer, ids[at:at + want.shape[0]])[0].cpu()
        if not torch.equal(got, want):
            raise ValueError(f"restored bytes of request {key}, {plane} differ from the snapshot")
        at += want.shape[0]
    if at != ids.numel():
        raise ValueError("restored row count differs from the snapshot")


def read_index_records(index_pool_layer, ids, *, page_tokens: int = 64, segment_bytes=(128, 4)):
    """Index records of logical ids from one layer's index page pool (uint8 [pages, 8448]: per page the
    keys of its 64 tokens, then their scales) -> uint8 [n, 132] (key bytes then scale bytes per record)."""
    import torch

    kb, sb = segment_bytes
    ids = ids.long()
    page, off = ids // page_tokens, ids % page_tokens
    cols_k = (off * kb).unsqueeze(1) + torch.arange(kb, device=ids.device)
    cols_s = (page_tokens * kb + off * sb).unsqueeze(1) + torch.arange(sb, device=ids.device)
    rows = index_pool_layer[page]
    return torch.cat([torch.gather(rows, 1, cols_k), torch.gather(rows, 1, cols_s)], dim=1).contiguous()


def write_index_records(index_pool_layer, ids, data, *, page_tokens: int = 64, segment_bytes=(128, 4)):
    """Inverse of :func:`read_index_records`; ``data`` uint8 [n, 132] (or bytes)."""
    import torch

    kb, sb = segment_bytes
    if isinstance(data, (bytes, bytearray)):
        data = torch.frombuffer(bytearray(data), dtype=torch.uint8).view(-1, kb + sb)
    data = data.to(index_pool_layer.device)
    ids = ids.long().to(index_pool_layer.device)
    page, off = ids // page_tokens, ids % page_tokens
    flat = index_pool_layer.view(-1)
    width = index_pool_layer.shape[1]
    base = page * width
    k_at = (base + off * kb).unsqueeze(1) + torch.arange(kb, device=ids.device)
    s_at = (base + page_tokens * kb + off * sb).unsqueeze(1) + torch.arange(sb, device=ids.device)
    flat[k_at.reshape(-1)] = data[:, :kb].reshape(-1)
    flat[s_at.reshape(-1)] = data[:, kb:].reshape(-1)
