"""A snapshot used as a KV bank: who restores what, the prefix tree over the restored requests, and the
speculative-decoding state that lets a restored request continue where it stopped.

* :func:`restore_routing` - for a snapshot written by ``S`` owners and a job of ``world`` ranks in a given
  layout, the list of (snapshot owner, request) shards every rank reads.  Pooled tensor parallelism stores a
  record on the rank that owns its page, so every rank reads every owner file and keeps its own records
  (the cache's writer routes by directory); data-parallel attention assigns whole requests to ranks
  round robin (or by an explicit placement) and a rank reads all owner files of its requests; replicated
  layouts read everything everywhere.
* :func:`rebuild_prefix_tree` - inserts every restored request's history into a radix tree under the pages
  it was restored to, so that later requests sharing a prefix reuse the restored records.
* :func:`save_continuation` / :func:`load_continuation` - the draft layer's inputs of a request (last hidden
  state, pending draft tokens, and selections stored as sequence POSITIONS so that they survive a change of
  logical ids), with a SHA-256 receipt.

Reference: ulacache/tools/snapshot/restore.py:96-349 (PreparedSequenceRestore, restore_public_request),
prefix.py:19-236 (stripe / save / restore of a prefix), speculative.py:9-79, cuda.py:53-649.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class RestoreShard:
    owner: int            # snapshot owner directory
    request: str          # request key
    keep: str             # "all" records of the shard, or "owned": the cache keeps those this rank owns


def restore_routing(owners: int, requests: Sequence[str], *, world: int, mode: str, kv_layout: str = "pooled",
                    placement: Optional[Dict[str, int]] = None) -> List[List[RestoreShard]]:
    """-> one shard list per rank.  ``placement`` (data-parallel attention): request key -> rank."""
    if owners < 1 or world < 1:
        raise ValueError("owners and world must be positive")
    if mode not in ("tp", "dpa"):
        raise ValueError("mode must be tp or dpa")
    plan: List[List[RestoreShard]] = [[] for _ in range(world)]
    if mode == "dpa":
        for i, key in enumerate(requests):
            rank = placement[key] if placement is not None else i % world
            if not 0 <= rank < world:
                raise ValueError(f"request {key} is placed on rank {rank} of {world}")
            plan[rank].extend(RestoreShard(o, key, "all") for o in range(owners))
        return plan
    keep = "owned" if (kv_layout == "pooled" and world > 1) else "all"
    for rank in range(world):
        plan[rank] = [RestoreShard(o, key, keep) for key in requests for o in range(owners)]
    return plan


def shard_positions(owner: int, owners: int, next_position: int) -> range:
    """Sequence positions stored in snapshot owner ``owner``'s files of a request."""
    return range(owner, next_position, owners)


def rebuild_prefix_tree(tree, requests, pages_of: Dict[str, Sequence[int]], *, page_tokens: int = 64) -> Dict[str, int]:
    """Insert every request's history (whole pages only) into ``tree`` (``serving.radix_tree.RadixPrefixTree``)
    under ``pages_of[key]``.  Returns key -> pages that were already cached by an earlier request (their
    restored copies are duplicates the caller may free)."""
    dup = {}
    for req in requests:
        hist = list(req.history_ids)
        whole = len(hist) // page_tokens
        pages = list(pages_of[req.key])[:whole]
        if len(pages) < whole:
            raise ValueError(f"request {req.key} has {whole} whole pages but {len(pages)} restored ones")
        dup[req.key] = len(tree.insert(hist[: whole * page_tokens], pages))
    return dup


CONTINUATION_FIELDS = ("hidden_state", "draft_tokens", "draft_probs", "bonus_token")


def save_continuation(path, *, hidden_state, draft_tokens=None, draft_probs=None, bonus_token=None,
                      selection_ids=None, request_ids=None) -> str:
    """Write one request's draft state; ``selection_ids`` (logical ids the draft layer selected last) are
    stored as positions within ``request_ids`` (the request's logical ids in sequence order).  The file must
    not exist.  Returns its SHA-256."""
    import torch

    data = dict(hidden_state=hidden_state.detach().cpu(),
                draft_tokens=None if draft_tokens is None else draft_tokens.detach().cpu(),
                draft_probs=None if draft_probs is None else draft_probs.detach().cpu(),
                bonus_token=None if bonus_token is None else bonus_token.detach().cpu(), selection_positions=None)
    if selection_ids is not None:
        if request_ids is None:
            raise ValueError("selections need the request's logical ids to become positions")
        rows = request_ids.detach().cpu().long()
        sel = selection_ids.detach().cpu().long()
        order = torch.argsort(rows)
        where = torch.searchsorted(rows[order], sel.clamp(min=0))
        valid = sel >= 0
        clipped = where.clamp(max=len(rows) - 1)
        if bool((valid & ((where >= len(rows)) | (rows[order][clipped] != sel))).any()):
            raise ValueError("a saved selection names a record outside the request's history")
        data["selection_positions"] = torch.where(valid, order[clipped], torch.full_like(sel, -1))
    path = Path(path)
    with path.open("xb") as f:
        torch.save(data, f)
    return hashlib.sha256(path.read_bytes()).hexdigest()


def load_continuation(path, expected_sha256: str, *, request_ids=None, device="cpu") -> dict:
    """Inverse of :func:`save_continuation`; positions are translated back through the restored request's
    logical ids (which may differ from the saved run's)."""
    import torch

    path = Path(path)
    if hashlib.sha256(path.read_bytes()).hexdigest() != expected_sha256:
        raise ValueError("the speculative continuation does not match its receipt")
    data = torch.load(path, map_location="cpu", weights_only=True)
    out = {k: (None if data[k] is None else data[k].to(device)) for k in CONTINUATION_FIELDS}
    pos = data.get("selection_positions")
    if pos is not None:
        if request_ids is None:
            raise ValueError("the continuation holds selections: pass the restored request's logical ids")
        rows = request_ids.detach().cpu().long()
        if bool((pos >= len(rows)).any()):
            raise ValueError("a saved selection lies beyond the restored history")
        ids = torch.where(pos >= 0, rows[pos.clamp(min=0)], torch.full_like(pos, -1))
        out["selection_ids"] = ids.to(device=device, dtype=torch.int32)
    else:
        out["selection_ids"] = None
    return out
