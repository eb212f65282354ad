"""Continuous-batching server loop around the model and the tiered cache, on one GPU or on several in
the data-parallel-attention layout (one process per GPU, requests dealt to the ranks; every rank keeps
its own cache, radix tree and scheduler and the ranks meet in the expert layers).

    srv = ServingEngine(cfg, max_batch=32, max_context=16384, device_records=..., host_records=...)
    srv.submit(request_id, prompt_token_ids, max_new_tokens, arrival_time)
    while srv.busy(): srv.step()
    srv.report()          # admitted requests, TTFT / TPOT percentiles, tokens/s, prefix reuse, tier traffic

One ``step`` decodes one token for every running request and, in the rows a prefill-sized step has
left, prefills the next chunk of one admitted request (decode never waits for a prompt).  Prefill reuses the decode kernels: the chunk's tokens are rows of a batch that all point at
the same request pages, with per-row context lengths (causal inside the chunk because every row's
KV and index key are written before any row is scored).  Finished prompts leave their whole pages in
the radix tree; a later request with the same prefix starts from them.  Admission charges a
request's whole history against ``device + host`` records; the cache decides which tier a record
lives in and promotes what sparse attention selects.

Several ranks: the expert exchange needs every rank in every layer with the same number of rows, so
the ranks agree on each step's row count over the CPU group (one small all-gather per step: a prefill
chunk anywhere makes it a ``prefill_chunk``-row step, otherwise ``max_batch`` rows) and fill up with
padding rows that write into a scratch page nobody reads.  The loop ends when no rank has work left.

Reference: the serving behaviour the reference gets from SGLang plus its adapters
(patches/sglang.patch:2144-2322 allocator, :8662-8836 admission, scripts/7_1_online/run.py metrics).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .admission import AdmissionController, CacheBudget
from .radix_tree import PAGE_TOKENS, RadixPrefixTree


@dataclass
class _Request:
    rid: int
    prompt: List[int]
    max_new: int
    arrival: float
    pages: List[int] = field(default_factory=list)       # logical pages in position order
    shared_pages: int = 0                                # leading pages borrowed from the radix tree
    nodes: list = field(default_factory=list)
    done_prompt: int = 0                                 # prompt tokens whose KV exists
    generated: List[int] = field(default_factory=list)
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    admit_time: Optional[float] = None


def percentile(values, p):
    if not values:
        return None
    s = sorted(values)
    k = min(len(s) - 1, max(0, int(round(p / 100.0 * (len(s) - 1)))))
    return s[k]


class ServingEngine:
    def __init__(self, cfg, *, max_batch: int, max_context: int, device_records: int, host_records: int = 0,
                 prefill_chunk: int = 512, device=None, seed: int = 0, clock=time.perf_counter,
                 rank: int = 0, world: int = 1, group=None, cpu_group=None):
        import torch
        from .. import client
        from ..bindings import LocalCacheBindings
        from ..cache.access import SparseAccessSpecification
        from ..cache.layers import LayerReuseSpecification
        from ..cache.specification import MemoryTierCapacity, UnifiedCacheSpecification
        from ..models.dsa_moe import DsaMoeModel
        from ..storage.layout import StorageLayout, record_plane

        self.cfg, self.clock = cfg, clock
        self.device = torch.device(device or "cuda")
        self.max_batch, self.chunk = max_batch, prefill_chunk
        self.rank, self.world, self.cpu_group = rank, world, cpu_group
        rows = max(max_batch, prefill_chunk)
        device_records = device_records // 64 * 64
        host_records = host_records // 64 * 64
        self.max_pages = (max_context + PAGE_TOKENS - 1) // PAGE_TOKENS
        spec = UnifiedCacheSpecification(
            storage_layout=StorageLayout(record_planes=(record_plane(cfg.kv_format),)),
            layer_reuse=LayerReuseSpecification.independent(cfg.layers),
            sparse_access=SparseAccessSpecification(rows, cfg.topk),
            capacity_plan=MemoryTierCapacity(device_record_capacity=device_records, host_record_capacity=host_records,
                                             maximum_write_record_count=1 << 20,
                                             maximum_residency_input_record_count=min(device_records, rows * (cfg.topk + 1))))
        self.cache = client.init(spec, LocalCacheBindings(device=self.device))
        total_pages = (device_records + host_records) // PAGE_TOKENS
        self.index_pool = torch.zeros((cfg.layers, total_pages + 2, 8448), dtype=torch.uint8, device=self.device)
        self.model = DsaMoeModel(cfg, device=self.device, cache=self.cache, index_pool=self.index_pool, tp=world, rank=rank,
                                 group=group, cpu_group=cpu_group, mode="dpa", max_batch=rows,
                                 max_context=max_context + 8, seed=seed)
        self._pad_page = None
        if world > 1:
            # padding rows of a step write their key / record into this page (position 0) and attend to it
            ids = self.cache.alloc(PAGE_TOKENS)
            self._pad_page = int(ids[0]) // PAGE_TOKENS
        self.admission = AdmissionController(CacheBudget(owners=1, device_records=device_records,
                                                         host_records=host_records, max_running_requests=max_batch))
        self.tree = RadixPrefixTree()
        self.waiting: List[_Request] = []
        self.prefilling: List[_Request] = []
        self.running: List[_Request] = []
        self.finished: List[_Request] = []
        self.stats = dict(prefill_tokens=0, reused_prefix_tokens=0, decode_steps=0, prefill_steps=0, decoded_tokens=0,
                          rejected=0)
        self._start = None

    # ------------------------------------------------------------------ requests --
    def submit(self, rid: int, prompt, max_new_tokens: int, arrival: Optional[float] = None):
        if len(prompt) + max_new_tokens > self.max_pages * PAGE_TOKENS:
            self.stats["rejected"] += 1
            return False
        self.waiting.append(_Request(rid, list(prompt), max_new_tokens, self.clock() if arrival is None else arrival))
        return True

    def busy(self) -> bool:
        """Work left on THIS rank (several ranks: keep calling ``step`` until it returns "done")."""
        return bool(self.waiting or self.prefilling or self.running)

    def _agree(self, want_rows: int, prefill: bool):
        """Several ranks: (rows every rank runs this step, whether any rank still has work)."""
        if self.world == 1:
            return want_rows, self.busy()
        import torch
        import torch.distributed as dist

        mine = torch.tensor([want_rows, int(prefill), int(self.busy())], dtype=torch.int64)
        every = [torch.zeros(3, dtype=torch.int64) for _ in range(self.world)]
        dist.all_gather(every, mine, group=self.cpu_group)
        every = torch.stack(every)
        if int(every[:, 2].sum()) == 0:
            return 0, False
        if int(every[:, 0].max()) == 0:
            return 0, True                                        # everybody is waiting for arrivals
        return (self.chunk if int(every[:, 1].max()) else self.max_batch), True

    def _alloc_pages(self, n: int) -> Optional[List[int]]:
        import torch

        if n == 0:
            return []
        ids = self.cache.alloc(n * PAGE_TOKENS)
        if ids is None:
            # give cached prefixes back to the pool and retry once
            freed = self.tree.evict(n)
            if freed:
                p = torch.tensor(freed, dtype=torch.int64, device=self.device)
                self.cache.free((p.unsqueeze(1) * PAGE_TOKENS + torch.arange(PAGE_TOKENS, device=self.device)).reshape(-1).to(torch.int32))
                ids = self.cache.alloc(n * PAGE_TOKENS)
            if ids is None:
                return None
        return (ids.view(-1, PAGE_TOKENS)[:, 0] // PAGE_TOKENS).tolist()

    def _admit(self, now: float):
        while self.waiting and self.waiting[0].arrival <= now:
            r = self.waiting[0]
            nodes = self.tree.match(r.prompt[:-1])               # the last prompt token is always recomputed
            reuse = len(nodes) * PAGE_TOKENS
            if not self.admission.can_admit(len(r.prompt), r.max_new, reusable_prefix=reuse,
                                            evictable_tokens=0):
                break
            need_pages = (len(r.prompt) + r.max_new + PAGE_TOKENS - 1) // PAGE_TOKENS - len(nodes)
            self.tree.lock(nodes)
            pages = self._alloc_pages(need_pages)
            if pages is None:
                self.tree.unlock(nodes)
                break
            self.admission.admit(r.rid, len(r.prompt), r.max_new, reusable_prefix=reuse)
            r.nodes, r.shared_pages = nodes, len(nodes)
            r.pages = [n.page for n in nodes] + pages
            r.done_prompt = reuse
            r.admit_time = now
            self.stats["reused_prefix_tokens"] += reuse
            self.waiting.pop(0)
            self.prefilling.append(r)

    # --------------------------------------------------------------------- steps --
    def _batch(self, rows):
        """rows: list of (request, input token, position) -> DecodeBatch on the device."""
        import torch
        from ..models.dsa_moe import DecodeBatch

        i32 = dict(dtype=torch.int32, device=self.device)
        tokens = torch.tensor([t for _, t, _ in rows], **i32)
        lengths = torch.tensor([p for _, _, p in rows], **i32)
        pad = getattr(self, "_pad_rows", 0)
        # one page-table row per distinct request, expanded to its rows (a prefill chunk is thousands of
        # rows of one request)
        order, index = {}, []
        for r, _, _ in rows:
            index.append(order.setdefault(id(r), len(order)))
        table = torch.full((len(order), self.max_pages), -1, dtype=torch.int32)
        seen = set()
        for r, _, _ in rows:
            k = order[id(r)]
            if k not in seen:
                seen.add(k)
                table[k, : len(r.pages)] = torch.tensor(r.pages, dtype=torch.int32)
        pages = table.to(self.device)[torch.tensor(index, device=self.device)] if rows else \
            torch.full((0, self.max_pages), -1, **i32)
        if pad:
            tokens = torch.cat([tokens, torch.zeros(pad, **i32)])
            lengths = torch.cat([lengths, torch.zeros(pad, **i32)])
            extra = torch.full((pad, self.max_pages), -1, **i32)
            extra[:, 0] = self._pad_page
            pages = torch.cat([pages, extra])
        return DecodeBatch(tokens=tokens, lengths=lengths, req_pages=pages, out_tokens=torch.zeros(tokens.numel(), **i32))

    def step(self):
        import torch

        now = self.clock()
        if self._start is None:
            self._start = now
        self._admit(now)
        # what this rank wants to run: one token for every running request, and - in the room a prefill-sized
        # step leaves beside them - the next chunk of the request being prefilled (decode never waits for a prompt)
        dec = [(r, r.generated[-1], len(r.prompt) + len(r.generated) - 1) for r in self.running]
        pre = []
        if self.prefilling:
            r = self.prefilling[0]
            lo = r.done_prompt
            hi = min(len(r.prompt), lo + max(0, self.chunk - len(dec)))
            pre = [(r, r.prompt[p], p) for p in range(lo, hi)]
        rows = dec + pre
        step_rows, anyone = self._agree(len(rows), bool(pre))
        if not anyone:
            return "done"
        if step_rows == 0:
            return "idle"
        if self.world > 1 and len(rows) > step_rows:
            raise RuntimeError("the agreed step is smaller than this rank's rows")
        self._pad_rows = step_rows - len(rows) if self.world > 1 else 0
        out = self.model.decode_step(self._batch(rows))
        self._pad_rows = 0
        t = None
        if dec:
            toks = out[: len(dec)].tolist()
            self.stats["decode_steps"] += 1
            self.stats["decoded_tokens"] += len(dec)
            for (r, _, _), tok in zip(dec, toks):
                r.generated.append(int(tok))
                if len(r.generated) >= r.max_new:
                    if t is None:
                        torch.cuda.synchronize()
                        t = self.clock()
                    r.finish_time = t
                    self.running.remove(r)
                    self._retire(r)
        if pre:
            r = self.prefilling[0]
            hi = r.done_prompt + len(pre)
            self.stats["prefill_tokens"] += len(pre)
            self.stats["prefill_steps"] += 1
            r.done_prompt = hi
            if hi == len(r.prompt):
                tok = int(out[len(rows) - 1])                     # sample of the last prompt position
                torch.cuda.synchronize()
                r.first_token_time = self.clock()
                r.generated.append(tok)
                self.prefilling.pop(0)
                if len(r.generated) < r.max_new:
                    self.running.append(r)
                else:
                    self._retire(r)
            return "prefill"
        if dec:
            return "decode"
        self.stats["padding_steps"] = self.stats.get("padding_steps", 0) + 1
        return "padding"                                          # only other ranks had rows

    def _retire(self, r: _Request):
        import torch

        if r.finish_time is None:
            r.finish_time = self.clock()
        self.tree.unlock(r.nodes)
        whole = len(r.prompt) // PAGE_TOKENS
        dup = self.tree.insert(r.prompt, r.pages[:whole])          # pages whose prefix got cached meanwhile
        keep = set(r.pages[:whole]) - set(dup)
        own = r.pages[r.shared_pages:]
        release = [p for p in own if p not in keep]
        if release:
            p = torch.tensor(release, dtype=torch.int64, device=self.device)
            ids = (p.unsqueeze(1) * PAGE_TOKENS + torch.arange(PAGE_TOKENS, device=self.device)).reshape(-1).to(torch.int32)
            self.cache.free(ids)
        self.admission.finish(r.rid)
        self.finished.append(r)

    # -------------------------------------------------------------------- report --
    def report(self) -> dict:
        fin = [r for r in self.finished if r.first_token_time is not None]
        ttft = [r.first_token_time - r.arrival for r in fin]
        tpot = [(r.finish_time - r.first_token_time) / max(1, len(r.generated) - 1) for r in fin if len(r.generated) > 1]
        wall = (max((r.finish_time for r in fin), default=self._start or 0) - (self._start or 0)) or 1e-9
        c = self.cache.counters()
        return {"admitted_requests": len(self.finished) + len(self.running) + len(self.prefilling),
                "finished_requests": len(fin), "rejected_requests": self.stats["rejected"],
                "ttft_s_p50": percentile(ttft, 50), "ttft_s_p99": percentile(ttft, 99),
                "tpot_s_p50": percentile(tpot, 50), "tpot_s_p99": percentile(tpot, 99),
                "output_tokens_per_s": sum(len(r.generated) for r in fin) / wall,
                "prefill_tokens": self.stats["prefill_tokens"], "reused_prefix_tokens": self.stats["reused_prefix_tokens"],
                "cached_prefix_pages": self.tree.cached_pages(), "decode_steps": self.stats["decode_steps"],
                "kv_token_capacity": self.admission.budget.token_capacity,
                "promotions": c.get("promotions", 0), "evictions": c.get("evictions", 0), "unserved": c.get("unserved", 0)}

    def close(self):
        heap = getattr(self.model, "comm_heap", None)
        if heap is not None:
            heap.close()
        self.cache.close()
