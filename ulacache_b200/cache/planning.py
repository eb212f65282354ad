"""Lowering of a :class:`LayerReuseSpecification` into the things an engine allocates:

* *storage banks*  - layers that share KV bytes share one bank (one plane per unique owner);
* *residency domains* - layers whose residency plan has one anchor share one directory / recency
  ring, the anchor runs the transaction and the followers reuse it;
* *selection producers* - the layer whose indexer output a layer consumes;
* *attention workspaces* - scratch for the gathered selection; domains whose layer intervals do not
  overlap share one (interval colouring).

Reference: ulacache/cache/planning.py:12 (PagedCacheExecutionPlan), :63, :92, :188;
storage/workspace.py:399 (workspace reuse colouring).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

from ..storage.workspace import AttentionWorkspaceLifetime, colour_workspaces
from .layers import LayerReuseSpecification


@dataclass(frozen=True)
class StorageBank:
    index: int
    owner_layer: int
    layers: Tuple[int, ...]


@dataclass(frozen=True)
class ResidencyDomain:
    index: int
    anchor_layer: int
    layers: Tuple[int, ...]
    banks: Tuple[int, ...]          # storage banks whose records move with this domain's plan
    workspace: int                  # attention workspace colour


@dataclass(frozen=True)
class PagedCacheExecutionPlan:
    banks: Tuple[StorageBank, ...]
    index_banks: Tuple[StorageBank, ...]
    domains: Tuple[ResidencyDomain, ...]
    selection_producer: Tuple[int, ...]      # per layer
    bank_of_layer: Tuple[int, ...]
    index_bank_of_layer: Tuple[int, ...]
    domain_of_layer: Tuple[int, ...]
    workspace_count: int
    selection_producers: Tuple[int, ...] = ()              # distinct producer layers, ascending
    selection_index_of_layer: Tuple[int, ...] = ()
    last_consumer_of_selection: Tuple[int, ...] = ()
    bank_ranges_of_domain: Tuple[Tuple[Tuple[int, int], ...], ...] = ()   # contiguous [first, last + 1) bank runs

    @property
    def step_reader_retirement_layer(self):
        """The layer after which ALL readers of a step can retire in one publication: the last consumer of any
        selection, provided every directory serves one selection per forward (None otherwise: retire per
        selection)."""
        domains = tuple(self.domain_of_layer[l] for l in self.selection_producers)
        if not domains or len(domains) != len(set(domains)):
            return None
        return max(self.last_consumer_of_selection)

    def is_anchor(self, layer: int) -> bool:
        return self.domains[self.domain_of_layer[layer]].anchor_layer == layer

    def followers(self, layer: int) -> Tuple[int, ...]:
        d = self.domains[self.domain_of_layer[layer]]
        return tuple(l for l in d.layers if l != d.anchor_layer)

    def describe(self) -> Dict[str, int]:
        return {"layers": len(self.bank_of_layer), "storage_banks": len(self.banks), "index_banks": len(self.index_banks),
                "residency_domains": len(self.domains), "attention_workspaces": self.workspace_count}


def _banks(owners) -> Tuple[Tuple[StorageBank, ...], Tuple[int, ...]]:
    uniq = sorted(set(owners))
    idx = {o: i for i, o in enumerate(uniq)}
    banks = tuple(StorageBank(i, o, tuple(l for l, ow in enumerate(owners) if ow == o)) for i, o in enumerate(uniq))
    return banks, tuple(idx[o] for o in owners)


def lower_layer_reuse(spec: LayerReuseSpecification) -> PagedCacheExecutionPlan:
    banks, bank_of = _banks(spec.key_value_storage_owners)
    ibanks, ibank_of = _banks(spec.index_storage_owners)
    anchors = sorted(set(spec.residency_plan_anchors))
    dom_idx = {a: i for i, a in enumerate(anchors)}
    dom_layers = {a: tuple(l for l, an in enumerate(spec.residency_plan_anchors) if an == a) for a in anchors}
    for a, layers in dom_layers.items():
        # a domain shares ONE selection: every layer of it must consume the same producer
        producers = {spec.sparse_selection_owners[l] for l in layers}
        if len(producers) != 1:
            raise ValueError(f"residency domain anchored at layer {a} mixes selections of layers {sorted(producers)}")
    lifetimes = [AttentionWorkspaceLifetime(dom_idx[a], min(ls), max(ls)) for a, ls in dom_layers.items()]
    colours, n_colours = colour_workspaces(lifetimes)
    domains = tuple(ResidencyDomain(dom_idx[a], a, dom_layers[a], tuple(sorted({bank_of[l] for l in dom_layers[a]})),
                                    colours[i]) for i, a in enumerate(anchors))
    producers = tuple(sorted(set(spec.sparse_selection_owners)))
    sel_idx = {l: i for i, l in enumerate(producers)}
    last = tuple(max(l for l, o in enumerate(spec.sparse_selection_owners) if o == pr) for pr in producers)
    ranges = []
    for d in domains:
        runs = []
        for b in d.banks:
            if runs and runs[-1][1] == b:
                runs[-1] = (runs[-1][0], b + 1)
            else:
                runs.append((b, b + 1))
        ranges.append(tuple(runs))
    return PagedCacheExecutionPlan(banks, ibanks, domains, tuple(spec.sparse_selection_owners), bank_of, ibank_of,
                                   tuple(dom_idx[a] for a in spec.residency_plan_anchors), n_colours, producers,
                                   tuple(sel_idx[o] for o in spec.sparse_selection_owners), last, tuple(ranges))


def lower_for_record_owners(spec: LayerReuseSpecification) -> PagedCacheExecutionPlan:
    """Lowering for the record-owner engine: every KV bank gets its OWN directory and publication boundary.  A
    selection shared across banks still names the same logical ids, but each bank plans its physical placement at
    its first consumer, so the selection owner of a layer becomes the first layer that consumes the same
    (bank, selection) pair; KV aliases stay in one bank.

    Reference: ulacache/cache/planning.py:63-90 (create_owner_paged_execution_plan)."""
    first = {}
    owners = []
    for layer, pair in enumerate(zip(spec.key_value_storage_owners, spec.sparse_selection_owners)):
        first.setdefault(pair, layer)
        owners.append(first[pair])
    lowered = LayerReuseSpecification(spec.key_value_storage_owners, spec.index_storage_owners, tuple(owners),
                                      spec.key_value_storage_owners)
    return lower_layer_reuse(lowered)


def validate_rank_local_specification(cache_specification) -> None:
    """Everything a rank-local engine cannot lower, refused before any memory is allocated: selections that do
    not name logical records, device capacity that is not page aligned, logical ids beyond int32, a shared KV
    bank or a shared selection that spans two directories.

    Reference: ulacache/cache/planning.py:92-186 (checks of create_paged_cache_execution_plan), :188-246
    (create_rank_local_layer_groups)."""
    reuse = cache_specification.layer_reuse
    access = cache_specification.sparse_access
    cap = cache_specification.capacity_plan
    layout = cache_specification.storage_layout
    if access.selection_unit != "record" or access.selection_identifier_space != "logical":
        raise NotImplementedError("selections must name canonical logical records")
    if cap.device_record_capacity % 64:
        raise ValueError("device record capacity must be a multiple of the 64-record page")
    if cap.logical_record_capacity >= 2 ** 31:
        raise ValueError("logical record ids must fit positive int32")
    for plane in layout.record_planes:
        if plane.bytes_per_record % 4:
            raise ValueError("records are multiples of 4 bytes")
    for layer, owner in enumerate(reuse.key_value_storage_owners):
        if reuse.residency_plan_anchors[layer] != reuse.residency_plan_anchors[owner]:
            raise NotImplementedError("a shared KV bank needs one residency directory")
    for layer, producer in enumerate(reuse.sparse_selection_owners):
        if reuse.residency_plan_anchors[layer] != reuse.residency_plan_anchors[producer]:
            raise NotImplementedError("a shared selection needs one residency directory")
    lower_layer_reuse(reuse)      # (also rejects a directory that would serve two selections in one forward)
