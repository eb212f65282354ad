"""On-disk format of a request KV snapshot ("KV bank"), file-compatible with the reference.

    <dir>/owner_NNN/requests.json.gz             this owner's copy of the metadata (layout + requests)
    <dir>/owner_NNN/request_RRRRR.<plane>.bin    one file per (request, plane): the owner's rows in position order
    <dir>/owner_NNN/SHARD.json                   the owner's receipt: metadata hash + size and SHA-256 of every file
    <dir>/COMMITTED.json                         written last: metadata hash + the hash of every owner's receipt

Planes are ``mla_<layer>`` (one KV record per owned token) and ``index_<layer>`` (index records,
key bytes then scale bytes) for the layers that anchor an index.  Ownership is by token position:
owner ``p % owners`` holds position ``p``.  The KV covers ``history_ids`` (prompt + generated minus
the last token); ``next_token_id`` is the token the restored request decodes next.

Commit protocol.  Every owner writes ONLY inside its own directory, which must not exist yet, so
owners in different processes never touch a common file.  ``finalize_snapshot`` (one caller, after
all owners finished) checks that every owner wrote the same metadata (byte-identical canonical
JSON, and the hash each receipt carries), that every receipt lists exactly the expected files with
the expected sizes, and only then writes ``COMMITTED.json``.  A directory that already holds a
``COMMITTED.json`` is never written into again.  Readers verify payload hashes by default
(``UDCACHE_SNAPSHOT_VERIFY_PAYLOAD=0`` opts out for repeated restores of a snapshot already verified).

Reference: ulacache/tools/snapshot/format.py (SnapshotLayout :44, SnapshotRequest :91,
SnapshotWriter :138, finalize_snapshot :217, SnapshotReader :237).  File names, JSON keys and the
``iter_plane(owner, request_key, plane)`` order follow it so that either library reads the other's
snapshots; ``index_anchors`` may be empty here (a cache without index planes), which the reference rejects.
"""
from __future__ import annotations

import gzip
import hashlib
import json
import os
from dataclasses import asdict, dataclass
from typing import Dict, Iterable, Iterator, Tuple

FORMAT = "ulacache-request-kv-v1"
OWNERSHIP = "token-position-modulo-owner-count"
STATE_NOTE = "KV covers history_ids; next_token_id is not yet in KV"
COMMIT_FILE = "COMMITTED.json"
RECEIPT_FILE = "SHARD.json"
METADATA_FILE = "requests.json.gz"


def canonical_json(value) -> bytes:
    """The byte string hashes are taken over: sorted keys, no whitespace."""
    return json.dumps(value, sort_keys=True, separators=(",", ":")).encode()


def sha256_hex(raw: bytes) -> str:
    return hashlib.sha256(raw).hexdigest()


def _publish(path: str, raw: bytes):
    """Write ``raw`` under a private temporary name (exclusive create), sync, then rename."""
    tmp = f"{path}.tmp"
    with open(tmp, "xb") as f:
        f.write(raw)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def owner_directory(path: str, owner: int) -> str:
    return os.path.join(path, f"owner_{owner:03d}")


def plane_file_name(request_index: int, plane: str) -> str:
    return f"request_{request_index:05d}.{plane}.bin"


@dataclass(frozen=True)
class SnapshotLayout:
    model_fingerprint: str
    owners: int
    layers: int
    mla_row_bytes: int
    index_anchors: Tuple[int, ...] = ()
    index_segment_bytes: Tuple[int, ...] = (128, 4)
    index_page_rows: int = 64
    kv_format: str = "mla.scaled656.fp8.v1"

    def __post_init__(self):
        object.__setattr__(self, "index_anchors", tuple(int(l) for l in self.index_anchors))
        object.__setattr__(self, "index_segment_bytes", tuple(int(w) for w in self.index_segment_bytes))
        if not isinstance(self.model_fingerprint, str) or not self.model_fingerprint:
            raise ValueError("A model / weight / format fingerprint is required")
        for name in ("owners", "layers", "mla_row_bytes", "index_page_rows"):
            v = getattr(self, name)
            if type(v) is not int or v < 1:
                raise ValueError(f"{name} must be a positive int")
        anchors = self.index_anchors
        if tuple(sorted(set(anchors))) != anchors or any(not 0 <= l < self.layers for l in anchors):
            raise ValueError("index_anchors must be unique, ascending and in range")
        if not self.index_segment_bytes or min(self.index_segment_bytes) < 1 or not self.kv_format:
            raise ValueError("Index segment widths and the KV format must be given")

    @property
    def index_row_bytes(self) -> int:
        return sum(self.index_segment_bytes)

    @property
    def index_layers(self) -> Tuple[int, ...]:
        return self.index_anchors

    def planes(self) -> Dict[str, int]:
        """Plane name -> bytes per row, in file order."""
        out = {f"mla_{l:03d}": self.mla_row_bytes for l in range(self.layers)}
        out.update({f"index_{l:03d}": self.index_row_bytes for l in self.index_anchors})
        return out

    @classmethod
    def from_json(cls, d: dict) -> "SnapshotLayout":
        return cls(**d)


@dataclass(frozen=True)
class SnapshotRequest:
    key: str
    input_ids: Tuple[int, ...]
    generated_ids: Tuple[int, ...]

    def __post_init__(self):
        object.__setattr__(self, "input_ids", tuple(int(t) for t in self.input_ids))
        object.__setattr__(self, "generated_ids", tuple(int(t) for t in self.generated_ids))
        if not isinstance(self.key, str) or not self.key:
            raise ValueError("A request key is required")
        if not self.input_ids or not self.generated_ids:
            raise ValueError("A snapshot request needs its prompt and at least the next token")
        if min(self.input_ids + self.generated_ids) < 0:
            raise ValueError("Token IDs must be non-negative")

    @property
    def history_ids(self) -> Tuple[int, ...]:
        return self.input_ids + self.generated_ids[:-1]

    @property
    def next_token_id(self) -> int:
        return self.generated_ids[-1]

    @property
    def next_position(self) -> int:
        return len(self.input_ids) + len(self.generated_ids) - 1

    def owned_rows(self, owner: int, owners: int) -> int:
        return len(range(owner, self.next_position, owners))


def snapshot_metadata(layout: SnapshotLayout, requests) -> dict:
    requests = tuple(requests)
    if not requests or len({r.key for r in requests}) != len(requests):
        raise ValueError("Snapshot requests must be non-empty with unique keys")
    return {"format": FORMAT, "layout": asdict(layout), "requests": [asdict(r) for r in requests],
            "ownership": OWNERSHIP, "state": STATE_NOTE}


def expected_files(layout: SnapshotLayout, requests, owner: int) -> Dict[str, Tuple[int, str, int]]:
    """File name -> (request index, plane, bytes) of everything one owner must write."""
    out = {}
    for i, req in enumerate(requests):
        rows = req.owned_rows(owner, layout.owners)
        for plane, width in layout.planes().items():
            out[plane_file_name(i, plane)] = (i, plane, rows * width)
    return out


class SnapshotWriter:
    """One owner's shard.  Touches nothing outside ``owner_NNN/``; the directory must be new."""

    def __init__(self, path: str, layout: SnapshotLayout, requests, owner: int):
        if type(owner) is not int or not 0 <= owner < layout.owners:
            raise ValueError("owner outside the layout")
        self.path, self.layout, self.owner = str(path), layout, owner
        self.requests = tuple(requests)
        self.metadata = snapshot_metadata(layout, self.requests)
        self._index_of = {r.key: i for i, r in enumerate(self.requests)}
        self._todo = expected_files(layout, self.requests, owner)
        self._done: Dict[str, dict] = {}
        os.makedirs(self.path, exist_ok=True)
        if os.path.exists(os.path.join(self.path, COMMIT_FILE)):
            raise FileExistsError("This directory holds a committed snapshot; it is never rewritten")
        self.dir = owner_directory(self.path, owner)
        os.mkdir(self.dir)                               # fails if this owner already wrote here
        _publish(os.path.join(self.dir, METADATA_FILE), gzip.compress(canonical_json(self.metadata), mtime=0))

    def write_plane(self, request_key: str, plane: str, chunks: Iterable[bytes]):
        """Write one request's rows of one plane from an iterable of byte chunks (position order)."""
        if request_key not in self._index_of or plane not in self.layout.planes():
            raise ValueError("Unknown request key or plane")
        name = plane_file_name(self._index_of[request_key], plane)
        if name in self._done:
            raise ValueError(f"{name} was already written")
        index, _, want = self._todo[name]
        got, digest = 0, hashlib.sha256()
        with open(os.path.join(self.dir, name), "xb") as f:
            for chunk in chunks:
                if not isinstance(chunk, (bytes, bytearray, memoryview)):
                    raise TypeError("Snapshot chunks must be raw bytes")
                got += len(chunk)
                if got > want:
                    raise ValueError(f"{name}: more bytes than its {want}-byte row range")
                f.write(chunk)
                digest.update(chunk)
            if got != want:
                raise ValueError(f"{name}: wrote {got} bytes, expected {want}")
            f.flush()
            os.fsync(f.fileno())
        self._done[name] = {"bytes": got, "sha256": digest.hexdigest(), "request_index": index, "plane": plane}

    def finish(self) -> dict:
        missing = sorted(set(self._todo) - set(self._done))
        if missing:
            raise ValueError(f"{len(missing)} plane files were not written (first: {missing[0]})")
        receipt = {"owner": self.owner, "metadata_sha256": sha256_hex(canonical_json(self.metadata)),
                   "files": self._done}
        _publish(os.path.join(self.dir, RECEIPT_FILE), canonical_json(receipt))
        return receipt


def _load_owner_metadata(path: str, owner: int) -> dict:
    with open(os.path.join(owner_directory(path, owner), METADATA_FILE), "rb") as f:
        return json.loads(gzip.decompress(f.read()))


def finalize_snapshot(path: str) -> dict:
    """Commit: every owner finished, all owners wrote identical metadata, every receipt is complete."""
    path = str(path)
    if os.path.exists(os.path.join(path, COMMIT_FILE)):
        raise FileExistsError("Snapshot already committed")
    reader = SnapshotReader(path, require_committed=False, verify_payload=False)
    receipts = {}
    for owner in range(reader.layout.owners):
        reader.validate_owner(owner)
        with open(os.path.join(owner_directory(path, owner), RECEIPT_FILE), "rb") as f:
            receipts[str(owner)] = sha256_hex(f.read())
    commit = {"format": reader.metadata["format"], "metadata_sha256": sha256_hex(canonical_json(reader.metadata)),
              "owners": receipts, "request_count": len(reader.requests)}
    _publish(os.path.join(path, COMMIT_FILE), canonical_json(commit))
    return commit


class SnapshotReader:
    def __init__(self, path: str, *, require_committed: bool = True, verify_payload=None):
        if verify_payload is None:
            setting = os.environ.get("UDCACHE_SNAPSHOT_VERIFY_PAYLOAD", "1")
            if setting not in ("0", "1"):
                raise ValueError("UDCACHE_SNAPSHOT_VERIFY_PAYLOAD must be 0 or 1")
            verify_payload = setting == "1"
        self.verify_payload = bool(verify_payload)
        self.path = str(path)
        self.metadata = _load_owner_metadata(self.path, 0)
        if self.metadata.get("format") != FORMAT or self.metadata.get("ownership") != OWNERSHIP:
            raise ValueError("Not a request KV snapshot of a supported format")
        self.layout = SnapshotLayout.from_json(self.metadata["layout"])
        self.requests = tuple(SnapshotRequest(**r) for r in self.metadata["requests"])
        if canonical_json(snapshot_metadata(self.layout, self.requests)) != canonical_json(self.metadata):
            raise ValueError("Snapshot metadata carries fields this version does not know")
        self._index_of = {r.key: i for i, r in enumerate(self.requests)}
        self._receipts: Dict[int, dict] = {}
        self.commit = None
        commit_path = os.path.join(self.path, COMMIT_FILE)
        if require_committed:
            if not os.path.exists(commit_path):
                raise ValueError("The snapshot was never committed")
            with open(commit_path, "rb") as f:
                self.commit = json.loads(f.read())
            if (self.commit.get("format") != FORMAT
                    or self.commit.get("metadata_sha256") != sha256_hex(canonical_json(self.metadata))
                    or set(self.commit.get("owners", {})) != {str(o) for o in range(self.layout.owners)}):
                raise ValueError("COMMITTED.json does not match the snapshot's metadata / owners")

    @property
    def committed(self) -> bool:
        return os.path.exists(os.path.join(self.path, COMMIT_FILE))

    def validate_owner(self, owner: int) -> dict:
        """Check one owner's metadata copy and receipt against the snapshot; returns the receipt."""
        if type(owner) is not int or not 0 <= owner < self.layout.owners:
            raise ValueError("owner outside the layout")
        if owner in self._receipts:
            return self._receipts[owner]
        d = owner_directory(self.path, owner)
        rpath = os.path.join(d, RECEIPT_FILE)
        if not os.path.exists(rpath):
            raise FileNotFoundError(f"owner {owner} has not finished its shard")
        with open(rpath, "rb") as f:
            raw = f.read()
        if self.commit is not None and sha256_hex(raw) != self.commit["owners"][str(owner)]:
            raise ValueError(f"owner {owner}: receipt differs from the committed one")
        receipt = json.loads(raw)
        want_hash = sha256_hex(canonical_json(self.metadata))
        if (receipt.get("owner") != owner or receipt.get("metadata_sha256") != want_hash
                or canonical_json(_load_owner_metadata(self.path, owner)) != canonical_json(self.metadata)):
            raise ValueError(f"owner {owner} wrote different request / layout metadata")
        want = expected_files(self.layout, self.requests, owner)
        if set(receipt["files"]) != set(want):
            raise ValueError(f"owner {owner}: receipt lists other files than the layout requires")
        for name, (index, plane, size) in want.items():
            rec = receipt["files"][name]
            if (rec["request_index"], rec["plane"], rec["bytes"]) != (index, plane, size):
                raise ValueError(f"owner {owner}: {name} does not match the layout")
            if os.path.getsize(os.path.join(d, name)) != size:
                raise ValueError(f"owner {owner}: {name} is truncated or extended")
        self._receipts[owner] = receipt
        return receipt

    def plane_file(self, owner: int, request_key: str, plane: str) -> str:
        if request_key not in self._index_of or plane not in self.layout.planes():
            raise ValueError("Unknown request key or plane")
        return os.path.join(owner_directory(self.path, owner), plane_file_name(self._index_of[request_key], plane))

    def plane_rows(self, owner: int, request_key: str) -> int:
        return self.requests[self._index_of[request_key]].owned_rows(owner, self.layout.owners)

    def iter_plane(self, owner: int, request_key: str, plane: str, *, chunk_bytes: int = 4 << 20,
                   verify_payload=None) -> Iterator[bytes]:
        """Chunks of one request's rows of one plane; the hash is checked when the iterator is
        exhausted (so a consumer must drain it before trusting the bytes)."""
        if chunk_bytes < 1:
            raise ValueError("chunk_bytes must be positive")
        verify = self.verify_payload if verify_payload is None else bool(verify_payload)
        receipt = self.validate_owner(owner)
        file_path = self.plane_file(owner, request_key, plane)
        rec = receipt["files"][os.path.basename(file_path)]
        digest, size = (hashlib.sha256() if verify else None), 0
        with open(file_path, "rb") as f:
            while True:
                chunk = f.read(chunk_bytes)
                if not chunk:
                    break
                size += len(chunk)
                if digest is not None:
                    digest.update(chunk)
                yield chunk
        if size != rec["bytes"] or (digest is not None and digest.hexdigest() != rec["sha256"]):
            raise ValueError(f"{os.path.basename(file_path)} of owner {owner}: checksum or size mismatch")

    def verify_plane(self, owner: int, request_key: str, plane: str) -> int:
        return sum(len(c) for c in self.iter_plane(owner, request_key, plane, verify_payload=True))

    def verify(self, *, chunk_bytes: int = 4 << 20) -> dict:
        """Re-hash every file of every owner; raises on the first mismatch."""
        total = 0
        for owner in range(self.layout.owners):
            for req in self.requests:
                for plane in self.layout.planes():
                    for chunk in self.iter_plane(owner, req.key, plane, chunk_bytes=chunk_bytes, verify_payload=True):
                        total += len(chunk)
        return {"format": FORMAT, "owners": self.layout.owners, "requests": len(self.requests), "verified_bytes": total}
