"""Record formats, page geometry and logical-ID arithmetic (pure Python).

These are the interchange facts of the cache: byte layouts of one KV record and
one index page, how logical record IDs are striped over owner ranks, and how a
directory entry encodes "HBM slot / host slot / unallocated".  The same constants
are mirrored in ``csrc/include/ulc/layout.h``; ``tests/test_layout.py`` keeps
the two in step.

Reference: ulacache/storage/layout.py (KeyValueRecordPlane :12, KeyValueStorageLayout :76,
history_capacity :124, NativePageLayout :139, record-major /
segment-major pages, NativeMLARecord :301, InterleavedRecordLayout :186,
PositionShardLayout :406) and ulacache/transfer/index_pages.py:12-15.
Nothing here imports torch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Tuple

PAGE_TOKENS = 64
PAGE_SHIFT = 6
LATENT_DIM = 512
ROPE_DIM = 64
SCALE_GROUP = 128
SCALE_GROUPS = LATENT_DIM // SCALE_GROUP
INDEX_DIM = 128
INDEX_RECORD_BYTES = 132
INDEX_PAGE_KEY_BYTES = PAGE_TOKENS * INDEX_DIM
INDEX_PAGE_BYTES = INDEX_PAGE_KEY_BYTES + PAGE_TOKENS * 4
MAX_TOPK = 2048
MAX_RANKS = 8
DIR_UNALLOCATED = -1
LOC_MASKED = -1


def dir_encode_host(slot: int) -> int:
    return -slot - 2


def dir_host_slot(entry: int) -> int:
    return -entry - 2


def loc_encode(rank: int, slot: int) -> int:
    return (rank << 28) | slot


def loc_decode(loc: int) -> Tuple[int, int]:
    return (loc >> 28) & 0x7, loc & 0x0FFFFFFF


@dataclass(frozen=True)
class KeyValueRecordPlane:
    """One plane of per-token records: a name, the byte length of each segment of
    a record, and whether a page stores records whole (record-major) or one
    segment after another (segment-major)."""

    name: str
    bytes_per_segment: Tuple[int, ...]
    native_encoding: str
    segment_major: bool = False
    page_tokens: int = PAGE_TOKENS
    page_alignment: int = 16

    def __post_init__(self):
        if not self.bytes_per_segment or any(b <= 0 for b in self.bytes_per_segment):
            raise ValueError("A record plane needs positive segment sizes")
        if self.page_tokens <= 0 or self.page_tokens & (self.page_tokens - 1):
            raise ValueError("Page size must be a power of two")
        if self.bytes_per_record % 4:
            raise ValueError("Records must be a multiple of 4 bytes")

    @property
    def bytes_per_record(self) -> int:
        return sum(self.bytes_per_segment)

    @property
    def bytes_per_page(self) -> int:
        raw = self.bytes_per_record * self.page_tokens
        a = self.page_alignment
        return (raw + a - 1) // a * a

    def record_offset(self, token_in_page: int, segment: int = 0) -> int:
        """Byte offset of a segment of a record inside its page."""
        if not 0 <= token_in_page < self.page_tokens:
            raise ValueError("Token outside the page")
        if self.segment_major:
            before = sum(self.bytes_per_segment[:segment]) * self.page_tokens
            return before + token_in_page * self.bytes_per_segment[segment]
        return token_in_page * self.bytes_per_record + sum(self.bytes_per_segment[:segment])


MLA_SCALED656 = KeyValueRecordPlane("mla", (528, 128), "mla.scaled656.fp8.v1")
MLA_RAW576 = KeyValueRecordPlane("mla", (576,), "mla.raw576.fp8.v1")
MLA_BF16 = KeyValueRecordPlane("mla", (1024, 128), "mla.bf16.1152.v1")
MLA_PACKED584 = KeyValueRecordPlane("mla", (576, 8), "mla.packed584.c4.v1", segment_major=True,
                                    page_alignment=576)
INDEX_FP8 = KeyValueRecordPlane("index", (128, 4), "index.fp8.132.v1", segment_major=True)

NATIVE_FORMATS = {p.native_encoding: p for p in (MLA_SCALED656, MLA_RAW576, MLA_BF16, MLA_PACKED584)}
FORMAT_ALIASES = {"scaled656": MLA_SCALED656, "raw576": MLA_RAW576, "bf16": MLA_BF16,
                  "packed584": MLA_PACKED584}
KERNEL_FORMAT_CODE = {"mla.scaled656.fp8.v1": 0, "mla.raw576.fp8.v1": 1, "mla.bf16.1152.v1": 2}


def native_mla_encodings_match(a: str, b: str) -> bool:
    return a == b and a in NATIVE_FORMATS


def record_plane(name_or_alias: str) -> KeyValueRecordPlane:
    if name_or_alias in FORMAT_ALIASES:
        return FORMAT_ALIASES[name_or_alias]
    if name_or_alias in NATIVE_FORMATS:
        return NATIVE_FORMATS[name_or_alias]
    raise ValueError(f"Unknown KV record format {name_or_alias!r}")


@dataclass(frozen=True)
class OwnerMap:
    """Striping of logical IDs over ``ranks`` owners in stripes of ``1 << stripe_shift``
    records (6 = whole 64-token pages, 0 = single tokens)."""

    ranks: int = 1
    stripe_shift: int = PAGE_SHIFT

    def __post_init__(self):
        if not 1 <= self.ranks <= MAX_RANKS:
            raise ValueError("Owner count must be between 1 and 8")
        if not 0 <= self.stripe_shift <= 16:
            raise ValueError("Stripe shift out of range")

    def owner(self, logical_id: int) -> int:
        return (logical_id >> self.stripe_shift) % self.ranks

    def local(self, logical_id: int) -> int:
        stripe = logical_id >> self.stripe_shift
        return ((stripe // self.ranks) << self.stripe_shift) | (logical_id & ((1 << self.stripe_shift) - 1))

    def to_global(self, owner: int, local_id: int) -> int:
        stripe = local_id >> self.stripe_shift
        return (((stripe * self.ranks) + owner) << self.stripe_shift) | (
            local_id & ((1 << self.stripe_shift) - 1))

    def local_count(self, logical_count: int) -> int:
        """Directory length an owner needs to cover logical IDs ``[0, logical_count)``."""
        stripe = 1 << self.stripe_shift
        stripes = (logical_count + stripe - 1) // stripe
        return ((stripes + self.ranks - 1) // self.ranks) * stripe

    @property
    def allocation_page(self) -> int:
        """Logical rows in one allocation unit that lands evenly on every owner."""
        return self.ranks * max(1 << self.stripe_shift, PAGE_TOKENS)


def history_capacity(max_queries: int, topk: int, multiplier: float, page_size: int = PAGE_TOKENS) -> int:
    """Resident history rows for ``max_queries`` queries of ``topk`` records with a reuse ``multiplier`` (>= 1):
    the product rounded up first to a whole row, then to whole pages, so that the ratio is never inflated by more
    than one page.  Must stay below 2^31 (slot indices are int32)."""
    import math

    if min(max_queries, topk, page_size) < 1:
        raise ValueError("Queries, top-k and page size are positive")
    if not math.isfinite(multiplier) or multiplier < 1:
        raise ValueError("The capacity multiplier is a finite number >= 1")
    rows = math.ceil(max_queries * topk * multiplier)
    slots = (rows + page_size - 1) // page_size * page_size
    if slots >= 2 ** 31:
        raise ValueError("Resident slots must fit int32 indices")
    return slots


@dataclass(frozen=True)
class NativePageLayout:
    """Byte geometry of a segment-major page as a transport sees it: ``page_size`` rows, each row split into
    ``segment_bytes`` segments that the page stores one segment array after another, the whole page padded to
    ``page_alignment``.  Segments and pages are multiples of 8 bytes (the unit record copies move)."""

    page_size: int
    segment_bytes: Tuple[int, ...]
    page_alignment: int = 1

    def __post_init__(self):
        object.__setattr__(self, "segment_bytes", tuple(self.segment_bytes))
        if self.page_size < 1 or self.page_alignment < 1:
            raise ValueError("Page size and alignment are positive")
        if not self.segment_bytes or any(w < 1 for w in self.segment_bytes):
            raise ValueError("A page row has at least one segment of positive width")
        if any(w % 8 for w in self.segment_bytes) or self.bytes_per_page % 8:
            raise ValueError("Segments and pages are multiples of 8 bytes")

    @classmethod
    def of_plane(cls, plane: "KeyValueRecordPlane") -> "NativePageLayout":
        return cls(plane.page_tokens, plane.bytes_per_segment if plane.segment_major else (plane.bytes_per_record,),
                   plane.page_alignment)

    @property
    def row_bytes(self) -> int:
        return sum(self.segment_bytes)

    @property
    def bytes_per_page(self) -> int:
        raw, a = self.page_size * self.row_bytes, self.page_alignment
        return (raw + a - 1) // a * a

    def byte_offset(self, row: int, byte: int) -> int:
        """Where byte ``byte`` of logical row ``row`` lives in a buffer of consecutive pages."""
        if row < 0 or not 0 <= byte < self.row_bytes:
            raise IndexError("Row or byte outside the geometry")
        page, in_page = divmod(row, self.page_size)
        row_before = page_before = 0
        for width in self.segment_bytes:
            if byte < row_before + width:
                return page * self.bytes_per_page + page_before + in_page * width + (byte - row_before)
            row_before += width
            page_before += self.page_size * width
        raise AssertionError("unreachable: byte < row_bytes")


@dataclass(frozen=True)
class InterleavedRecordLayout:
    """Owner-striped pool geometry: how many slots each owner holds in HBM and in
    host memory, and the logical capacity that results."""

    owners: OwnerMap
    device_slots_per_owner: int
    host_slots_per_owner: int = 0

    def __post_init__(self):
        for v in (self.device_slots_per_owner, self.host_slots_per_owner):
            if v < 0 or v % PAGE_TOKENS:
                raise ValueError("Slot counts must be non-negative multiples of the page size")
        if self.slots_per_owner * self.owners.ranks >= 2 ** 31:
            raise ValueError("Logical capacity must fit int32 IDs")

    @property
    def slots_per_owner(self) -> int:
        return self.device_slots_per_owner + self.host_slots_per_owner

    @property
    def logical_capacity(self) -> int:
        """Usable logical IDs; ID 0 is reserved as padding."""
        return self.slots_per_owner * self.owners.ranks

    @property
    def directory_length(self) -> int:
        return self.owners.local_count(self.logical_capacity + self.owners.allocation_page)


@dataclass(frozen=True)
class PositionShardLayout:
    """Context-parallel sharding: token position ``p`` of a request lives on rank
    ``p % ranks`` at local position ``p // ranks``."""

    ranks: int

    def owner(self, position: int) -> int:
        return position % self.ranks

    def local(self, position: int) -> int:
        return position // self.ranks

    def local_length(self, length: int, rank: int) -> int:
        return (length - rank + self.ranks - 1) // self.ranks if length > rank else 0


@dataclass(frozen=True)
class StorageLayout:
    """Everything a cache instance stores per token: the record planes (normally
    one MLA plane) and whether an index plane rides along."""

    record_planes: Tuple[KeyValueRecordPlane, ...] = (MLA_SCALED656,)
    index_plane: KeyValueRecordPlane | None = None
    layer_begin: int = 0
    layer_end: int | None = None
    planes_by_name: dict = field(default_factory=dict, compare=False, repr=False)
    name: str = "kv"
    record_kind: str = "token"           # "token": one record per token; "compressed": one per tokens_per_record tokens
    tokens_per_record: int = 1

    def __post_init__(self):
        if not self.record_planes:
            raise ValueError("At least one record plane is required")
        if not self.name:
            raise ValueError("A storage tier has a name")
        if self.record_kind not in ("token", "compressed"):
            raise ValueError("record_kind is token or compressed")
        if type(self.tokens_per_record) is not int or self.tokens_per_record < 1:
            raise ValueError("tokens_per_record is a positive integer")
        if self.record_kind == "token" and self.tokens_per_record != 1:
            raise ValueError("A token record stands for exactly one token")
        if len({p.page_tokens for p in self.record_planes}) != 1:
            raise ValueError("The planes of one tier share one page size")
        object.__setattr__(self, "planes_by_name", {p.name: p for p in self.record_planes})

    @property
    def bytes_per_token(self) -> int:
        return sum(p.bytes_per_record for p in self.record_planes)

    @property
    def bytes_per_record(self) -> int:
        return self.bytes_per_token

    @property
    def records_per_page(self) -> int:
        return self.record_planes[0].page_tokens

    def calculate_storage_bytes(self, records: int) -> int:
        """Bytes that ``records`` records occupy in every plane, page padding of a partly used page included."""
        if type(records) is not int or records < 0:
            raise ValueError("Record count is a non-negative integer")
        pages = (records + self.records_per_page - 1) // self.records_per_page
        return pages * sum(p.bytes_per_page for p in self.record_planes)


KeyValueStorageLayout = StorageLayout        # the name the reference exports for a storage tier


@dataclass(frozen=True)
class PackedMLARecordSpec:
    """What a model's cache adapter declares about a packed, indexed MLA tier, so that the planner needs to know
    neither the model family nor the packing: which layers keep such records, each layer's Index anchor (layers of
    one group share the anchor's selection), the full selected width the attention kernel consumes (multiples of
    256, any appended tail included), the row's bytes and segments, and the padding a kernel ABI puts on every page.

    Reference: ulacache/storage/layout.py:352-404 (``FlowKVPackedMLASpec``, exported as ``RecordSpec``)."""

    compression_ratio: int
    indexed_layer_ids: Tuple[int, ...]
    topk: int
    row_bytes: int
    native_segment_bytes: Tuple[int, ...]
    index_layer_anchors: Tuple[int, ...]
    page_storage_alignment: int = 1

    def __post_init__(self):
        for name in ("indexed_layer_ids", "native_segment_bytes", "index_layer_anchors"):
            object.__setattr__(self, name, tuple(getattr(self, name)))
        if self.topk <= 0 or self.topk % 256:
            raise NotImplementedError(f"the selected width must be a positive multiple of 256, not {self.topk}")
        if self.compression_ratio < 1 or self.page_storage_alignment < 1:
            raise ValueError("Compression ratio and page alignment are positive")
        if sum(self.native_segment_bytes) != self.row_bytes or any(w < 1 for w in self.native_segment_bytes):
            raise ValueError("The segments must add up to the row")
        if len(self.index_layer_anchors) != len(self.indexed_layer_ids):
            raise ValueError("Every indexed layer names its Index anchor")
        if len(set(self.indexed_layer_ids)) != len(self.indexed_layer_ids):
            raise ValueError("An indexed layer appears once")
        if not set(self.index_layer_anchors) <= set(self.indexed_layer_ids):
            raise ValueError("An Index anchor is itself an indexed layer")

    def _local(self, start_layer: int, end_layer: int) -> Tuple[int, ...]:
        if start_layer < 0 or end_layer <= start_layer:
            raise ValueError("Invalid layer range")
        return tuple(l for l in self.indexed_layer_ids if start_layer <= l < end_layer)

    def local_layer_count(self, start_layer: int, end_layer: int) -> int:
        return len(self._local(start_layer, end_layer))

    def local_layer_anchors(self, start_layer: int, end_layer: int) -> Tuple[int, ...]:
        """For the indexed layers of a pipeline stage, in order: the stage-local position of each one's anchor.
        A selection group may not straddle the stage boundary."""
        mine = self._local(start_layer, end_layer)
        position = {layer: i for i, layer in enumerate(mine)}
        anchor_of = dict(zip(self.indexed_layer_ids, self.index_layer_anchors))
        if any(anchor_of[l] not in position for l in mine):
            raise ValueError("A shared-Index group crosses the stage boundary")
        return tuple(position[anchor_of[l]] for l in mine)

    def plane(self, name: str = "mla", native_encoding: str = "mla.packed.v1", page_tokens: int = PAGE_TOKENS
              ) -> KeyValueRecordPlane:
        """The tier's record plane: segment-major pages when the row has more than one segment."""
        return KeyValueRecordPlane(name, self.native_segment_bytes, native_encoding,
                                   segment_major=len(self.native_segment_bytes) > 1, page_tokens=page_tokens,
                                   page_alignment=self.page_storage_alignment)

    def storage_layout(self, name: str = "packed") -> StorageLayout:
        kind = "compressed" if self.compression_ratio > 1 else "token"
        return StorageLayout(record_planes=(self.plane(),), name=name, record_kind=kind,
                             tokens_per_record=self.compression_ratio)


RecordSpec = PackedMLARecordSpec
