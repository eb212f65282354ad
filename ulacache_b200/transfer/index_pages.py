"""Direct-receive plans for index pages (8448-byte pages: 64 fp8 keys of 128 + 64 fp32 scales).

A request's index entries arrive as whole pages; the last page of a prompt may be partial and is
then sent as keys [0, n) and scales [0, n) separately.

Reference: ulacache/transfer/index_pages.py:1-184, owner_index_receive.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

PAGE_TOKENS = 64
KEY_BYTES = 128
PAGE_KEY_BYTES = PAGE_TOKENS * KEY_BYTES
PAGE_BYTES = PAGE_KEY_BYTES + PAGE_TOKENS * 4


def plan_index_page_receive(pages, tokens: int, *, base_address: int, layer_stride: int, layers: int,
                            ranks: int = 1, rank: int = 0) -> List[List[Tuple[int, int]]]:
    """(address, bytes) extents per layer for the index pages THIS rank owns of a request with
    ``tokens`` tokens.  ``pages``: physical page per allocation page of the request (owner-local)."""
    out = []
    for layer in range(layers):
        base = base_address + layer * layer_stride
        ext = []
        for a, phys in enumerate(pages):
            first = (a * ranks + rank) * PAGE_TOKENS
            n = max(0, min(PAGE_TOKENS, tokens - first))
            if n == 0 or phys < 0:
                continue
            addr = base + int(phys) * PAGE_BYTES
            if n == PAGE_TOKENS:
                ext.append((addr, PAGE_BYTES))
            else:
                ext.append((addr, n * KEY_BYTES))
                ext.append((addr + PAGE_KEY_BYTES, n * 4))
        out.append(ext)
    return out


# ----------------------------------------------------------------------------------------------
# Record-level publication of received Index entries.
#
# A prefill worker delivers Index entries into a STAGING buffer of native pages (64 keys of 128
# fp8 bytes, then 64 fp32 scales: a page is not an array of 132-byte records).  Publication pairs
# every received record with its canonical destination on the owner - logical record r belongs to
# page r >> 6, pages are striped over the owners (owner = page % ranks, owner-local page =
# page // ranks) - and copies key and scale separately.  The whole plan is validated before a byte
# moves; a destination is written at most once; staging and canonical storage must not alias; the
# caller vouches that the transport has retired its writes.
#
# Reference: ulacache/transfer/index_pages.py:19-184 (IndexRecordCopy, plan_index_record_copies,
# publish_index_record_bytes, validate_index_record_plan).  The reference stripes single records
# over the owners; here ownership is by 64-record page, as everywhere in this package.
# ----------------------------------------------------------------------------------------------
SCALE_BYTES = 4


def record_offsets(record: int) -> Tuple[int, int]:
    """(byte offset of the key, byte offset of the scale) of ``record`` in a buffer of native pages."""
    page, off = divmod(record, PAGE_TOKENS)
    base = page * PAGE_BYTES
    return base + off * KEY_BYTES, base + PAGE_KEY_BYTES + off * SCALE_BYTES


def owner_local_record(logical_record: int, ranks: int) -> Tuple[int, int]:
    """(owner rank, owner-local record) of a logical Index record under page striping."""
    page, off = divmod(logical_record, PAGE_TOKENS)
    return page % ranks, (page // ranks) * PAGE_TOKENS + off


@dataclass(frozen=True)
class IndexRecordCopy:
    ranks: int
    rank: int
    logical_record: int
    received_record: int
    destination_record: int
    source_key_byte: int
    destination_key_byte: int
    source_scale_byte: int
    destination_scale_byte: int

    def __post_init__(self):
        if any(type(v) is not int for v in vars(self).values()):
            raise ValueError("Index record coordinates must be integers")
        owner, local = owner_local_record(self.logical_record, max(self.ranks, 1))
        if (self.ranks < 1 or not 0 <= self.rank < self.ranks or self.logical_record < self.ranks * PAGE_TOKENS
                or owner != self.rank or local != self.destination_record or self.received_record < 0
                or (self.source_key_byte, self.source_scale_byte) != record_offsets(self.received_record)
                or (self.destination_key_byte, self.destination_scale_byte) != record_offsets(self.destination_record)):
            raise ValueError("Index record plan disagrees with the owner / page coordinates")


def plan_index_record_copies(logical_records, received_records, *, ranks: int, rank: int):
    """Copies for the records THIS rank owns.  ``logical_records[i]`` arrived as staging record
    ``received_records[i]``.  The first allocation page of every owner (logical records below ``ranks * 64``) is
    padding and never a destination."""
    if type(ranks) is not int or ranks < 1 or type(rank) is not int or not 0 <= rank < ranks:
        raise ValueError("Index ownership needs a positive owner count and a rank inside it")
    logical, received = tuple(logical_records), tuple(received_records)
    if len(logical) != len(received):
        raise ValueError("logical and received Index record counts differ")
    if any(type(r) is not int or r < ranks * PAGE_TOKENS for r in logical) or any(type(r) is not int or r < 0 for r in received):
        raise ValueError("Index records exclude padding and negative receive rows")
    if len(set(logical)) != len(logical) or len(set(received)) != len(received):
        raise ValueError("Index transfer records must be unique")
    out = []
    for lr, rr in zip(logical, received):
        owner, local = owner_local_record(lr, ranks)
        if owner != rank:
            continue
        sk, ss = record_offsets(rr)
        dk, ds = record_offsets(local)
        out.append(IndexRecordCopy(ranks, rank, lr, rr, local, sk, dk, ss, ds))
    return tuple(out)


def validate_index_record_plan(plan, source_bytes: int, destination_bytes: int):
    """Everything that can be wrong with a plan, checked before publication starts."""
    if any(type(n) is not int or n < 0 or n % PAGE_BYTES for n in (source_bytes, destination_bytes)):
        raise ValueError("Index storage holds complete native pages")
    plans = tuple(plan)
    if any(type(p) is not IndexRecordCopy for p in plans):
        raise ValueError("Index publication takes validated record plans")
    if len({(p.ranks, p.rank) for p in plans}) > 1:
        raise ValueError("one Index bank has one owner layout")
    if len({p.destination_record for p in plans}) != len(plans):
        raise ValueError("Index publication cannot write a destination twice")
    for p in plans:
        if p.destination_record < PAGE_TOKENS:
            raise ValueError("the owner's first page is padding, not a destination")
        for start, width, cap in ((p.source_key_byte, KEY_BYTES, source_bytes), (p.source_scale_byte, SCALE_BYTES, source_bytes),
                                  (p.destination_key_byte, KEY_BYTES, destination_bytes),
                                  (p.destination_scale_byte, SCALE_BYTES, destination_bytes)):
            if start < 0 or start + width > cap:
                raise ValueError("an Index record copy exceeds its storage")
    return plans


def publish_index_record_bytes(source, destination, plan, *, transport_quiesced) -> int:
    """Host form (and byte oracle of the device form): copy keys and scales of ``plan`` from the staging buffer
    to canonical storage (objects with the buffer protocol).  Returns the number of records published."""
    if transport_quiesced is not True:
        raise RuntimeError("Index publication needs the transport's writes retired")
    src, dst = memoryview(source), memoryview(destination)
    if not src.c_contiguous or not dst.c_contiguous:
        raise ValueError("Index page buffers must be contiguous")
    if src.obj is dst.obj:
        raise ValueError("receive staging and canonical Index storage must not alias")
    src, dst = src.cast("B"), dst.cast("B")
    if dst.readonly:
        raise ValueError("canonical Index storage must be writable")
    plans = validate_index_record_plan(plan, src.nbytes, dst.nbytes)
    for p in plans:
        dst[p.destination_key_byte:p.destination_key_byte + KEY_BYTES] = src[p.source_key_byte:p.source_key_byte + KEY_BYTES]
        dst[p.destination_scale_byte:p.destination_scale_byte + SCALE_BYTES] = \
            src[p.source_scale_byte:p.source_scale_byte + SCALE_BYTES]
    return len(plans)


def publish_index_records(source_pages, destination_pages, plan, *, transport_quiesced) -> int:
    """Tensor form (CPU or CUDA uint8 tensors of whole pages, any leading shape): two gathers and two scatters
    over all records of the plan."""
    import torch

    if transport_quiesced is not True:
        raise RuntimeError("Index publication needs the transport's writes retired")
    src, dst = source_pages.reshape(-1), destination_pages.reshape(-1)
    if src.dtype != torch.uint8 or dst.dtype != torch.uint8 or not source_pages.is_contiguous() or not destination_pages.is_contiguous():
        raise ValueError("Index page buffers are contiguous uint8 tensors")
    if src.untyped_storage().data_ptr() == dst.untyped_storage().data_ptr():
        raise ValueError("receive staging and canonical Index storage must not alias")
    plans = validate_index_record_plan(plan, int(src.numel()), int(dst.numel()))
    if not plans:
        return 0
    dev = dst.device
    sk = torch.tensor([p.source_key_byte for p in plans], device=dev)[:, None] + torch.arange(KEY_BYTES, device=dev)
    dk = torch.tensor([p.destination_key_byte for p in plans], device=dev)[:, None] + torch.arange(KEY_BYTES, device=dev)
    ss = torch.tensor([p.source_scale_byte for p in plans], device=dev)[:, None] + torch.arange(SCALE_BYTES, device=dev)
    ds = torch.tensor([p.destination_scale_byte for p in plans], device=dev)[:, None] + torch.arange(SCALE_BYTES, device=dev)
    dst[dk.reshape(-1)] = src[sk.reshape(-1)]
    dst[ds.reshape(-1)] = src[ss.reshape(-1)]
    return len(plans)
