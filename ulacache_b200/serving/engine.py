"""Decode engine: the call a user makes to run the model against the pooled cache.

    eng = DecodeEngine(cfg, batch=16, prompt_len=32768, max_new_tokens=1024)   # one process per GPU
    eng.fill_synthetic()                    # stands in for prefill: random KV + index entries
    for _ in range(n):
        next_tokens = eng.step(host_tokens) # pinned host int32 [B] in, pinned host int32 [B] out

``step`` copies the step's input tokens host -> device, replays the captured decode
graph (every kernel of every layer, the cache transaction included) and copies the
sampled tokens device -> host.  ``step_device`` skips the two copies and feeds each
step with the previous step's samples.

The reference library leaves this role to the serving framework it patches
(scripts/decode.py there drives a running server over HTTP and measures a steady
decode window after a separate fill phase; the same split is kept here).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineGeometry:
    batch: int                  # requests decoded by THIS rank's model (tp: global batch)
    tokens_per_request: int     # prompt + generated, rounded to the allocation page
    alloc_pages_per_request: int
    slots_per_rank: int
    index_pages: int


def init_distributed():
    """(rank, world, local_rank, device_group, cpu_group) from the torchrun environment."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1:
        return 0, 1, 0, None, None
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    if not dist.is_initialized():
        # The collective library prints its version banner on STDOUT while it creates its first communicator (at
        # the VERSION debug level whatever NCCL_DEBUG_FILE says).  Programs that print a result line on stdout must
        # not have it mixed in: file descriptor 1 points at stderr while the communicator comes up.
        import sys

        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()                     # the first collective: the communicator exists afterwards
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    cpu_group = dist.new_group(backend="gloo")
    return rank, world, local, dist.group.WORLD, cpu_group


class DecodeEngine:
    def __init__(self, cfg, *, batch: int, prompt_len: int, max_new_tokens: int, mode: str = "tp",
                 rank: int = 0, world: int = 1, local_rank: int = 0, group=None, cpu_group=None,
                 host_record_capacity: int = 0, device_record_capacity: Optional[int] = None,
                 use_graph: bool = True, seed: int = 0,
                 kv_transport: str = "auto", comm: str = "peer", spec_steps: int = 3, force_accept=None,
                 tp_attention: str = "owner", weights_from_full: bool = False, kv_layout: str = "pooled"):
        import torch
        from .. import client
        from ..bindings import LocalCacheBindings, TensorParallelCacheBindings
        from ..cache.access import SparseAccessSpecification
        from ..cache.layers import LayerReuseSpecification
        from ..cache.specification import MemoryTierCapacity, UnifiedCacheSpecification
        from ..models.dsa_moe import DecodeBatch, DsaMoeModel
        from ..storage.layout import StorageLayout, record_plane

        self.cfg, self.mode, self.rank, self.world = cfg, mode, rank, world
        self.device = torch.device("cuda", local_rank)
        torch.cuda.set_device(self.device)
        kv_ranks = world if (mode == "tp" and kv_layout == "pooled") else 1
        self.kv_ranks, self.kv_layout = kv_ranks, kv_layout
        span = 64 * kv_ranks
        # speculative decoding: rows per request in the verify pass, and room for rejected drafts
        self.spec_steps = spec_steps if cfg.mtp_layers else 0
        self.force_accept = force_accept
        rows_per_request = self.spec_steps + 1
        total = (prompt_len + max_new_tokens * rows_per_request + rows_per_request + span - 1) // span * span
        pages = total // span
        # every owner holds total / kv_ranks tokens of every request
        needed = (batch * total // kv_ranks + 64 + 63) // 64 * 64
        # With a host tier the records of a rank are split between HBM slots and pinned host slots
        # (``device_record_capacity`` + ``host_record_capacity`` must hold all of them); promotions and
        # evictions then run inside every decode step.
        slots = needed if device_record_capacity is None else (int(device_record_capacity) + 63) // 64 * 64
        if slots + host_record_capacity < needed:
            raise ValueError(f"{needed} records per rank are needed, the tiers hold {slots} + {host_record_capacity}")
        self.records_needed = needed
        self.geometry = EngineGeometry(batch, total, pages, slots, batch * pages + 2)
        self.prompt_len, self.max_new_tokens = prompt_len, max_new_tokens
        plane = record_plane(cfg.kv_format)
        spec = UnifiedCacheSpecification(
            storage_layout=StorageLayout(record_planes=(plane,)),
            layer_reuse=LayerReuseSpecification.independent(cfg.cache_layers),
            sparse_access=SparseAccessSpecification(batch * rows_per_request, cfg.topk),
            capacity_plan=MemoryTierCapacity(device_record_capacity=slots, host_record_capacity=host_record_capacity,
                                             maximum_write_record_count=1 << 20,
                                             maximum_residency_input_record_count=min(slots, batch * rows_per_request * (cfg.topk + 1))))
        if kv_ranks > 1:
            bindings = TensorParallelCacheBindings(device=self.device, process_group=cpu_group, rank=rank,
                                                   world_size=world, transport=kv_transport)
        else:
            bindings = LocalCacheBindings(device=self.device)
        self.cache = client.init(spec, bindings)
        self.index_pool = torch.zeros((cfg.cache_layers, self.geometry.index_pages, 8448), dtype=torch.uint8, device=self.device)
        self.model = DsaMoeModel(cfg, device=self.device, cache=self.cache, index_pool=self.index_pool, tp=world,
                                 rank=rank, group=group, cpu_group=cpu_group, mode=mode, max_batch=batch * rows_per_request,
                                 max_context=total + 8, seed=seed, comm=comm, tp_attention=tp_attention,
                                 weights_from_full=weights_from_full, kv_layout=kv_layout)
        i32 = dict(dtype=torch.int32, device=self.device)
        self.batch = DecodeBatch(tokens=torch.zeros(batch, **i32), lengths=torch.zeros(batch, **i32),
                                 req_pages=torch.full((batch, pages), -1, **i32), out_tokens=torch.zeros(batch, **i32))
        self.spec = None
        if self.spec_steps:
            from ..models.dsa_moe import SpeculativeBatch

            self.spec = SpeculativeBatch(tokens=self.batch.tokens, lengths=self.batch.lengths, req_pages=self.batch.req_pages,
                                         drafts=torch.zeros((batch, self.spec_steps), **i32),
                                         out=torch.zeros((batch, self.spec_steps + 1), **i32),
                                         accepted=torch.zeros(batch, **i32),
                                         emitted=torch.zeros(1, dtype=torch.int64, device=self.device))
        self.host_in = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self.host_out = torch.zeros(batch, dtype=torch.int32).pin_memory()
        self.use_graph = use_graph
        self.graph = None
        self.launches_per_step = 0
        self.steps_done = 0
        self._ids = None

    # ------------------------------------------------------------------- fill --
    def fill_synthetic(self, chunk: int = 32768, seed: int = 1, on_chunk=None):
        """Admit ``batch`` requests with ``prompt_len`` cached tokens each: allocate their
        logical IDs, then write random KV records and index keys for every layer through
        the cache's own writers (the decode measurement starts from a full cache, as a
        restore from a KV snapshot would leave it).  ``on_chunk(layer, first, last, latent, rope,
        index_key)`` sees what was written for tokens ``first..last`` of the request-major token list
        (for oracles that keep their own copy of the history)."""
        import torch
        from ..ops import records

        g = self.geometry
        span = 64 * self.kv_ranks
        gen = torch.Generator(device=self.device).manual_seed(seed)
        all_ids = []
        for r in range(g.batch):
            ids = self.cache.alloc(g.tokens_per_request)
            pages = (ids.view(-1, span)[:, 0] // span).to(torch.int32)
            if int(pages.max()) >= g.index_pages:
                raise MemoryError("index pool too small for the allocated pages")
            self.batch.req_pages[r] = pages
            all_ids.append(ids[: self.prompt_len])
        self.request_ids = all_ids                       # logical record IDs of every request's prompt, in order
        self.batch.lengths.fill_(self.prompt_len)
        self.batch.tokens.copy_(torch.randint(0, self.cfg.vocab, (g.batch,), device=self.device, generator=gen).to(torch.int32))
        ids = torch.cat(all_ids)
        positions = torch.arange(self.prompt_len, device=self.device, dtype=torch.int32).repeat(g.batch)
        n = ids.numel()
        for layer in range(self.cfg.cache_layers):
            for s in range(0, n, chunk):
                e = min(n, s + chunk)
                lat = torch.randn(e - s, 512, device=self.device, generator=gen, dtype=torch.bfloat16)
                rope = torch.randn(e - s, 64, device=self.device, generator=gen, dtype=torch.bfloat16)
                self.cache.write(ids[s:e], layer, (lat, rope))
                k = torch.randn(e - s, 128, device=self.device, generator=gen, dtype=torch.bfloat16)
                records.index_key_store(self.model.index_views[layer], k, ids[s:e], owner_only=True,
                                        status=self.model.status)
                if on_chunk is not None:
                    on_chunk(layer, s, e, lat, rope, k)
        torch.cuda.synchronize()
        self.cache.check("synthetic fill")

    # ------------------------------------------------------------------- step --
    def _decode_once(self):
        if self.spec is not None:
            self.model.speculative_step(self.spec, self.force_accept)
            self.batch.out_tokens.copy_(self.batch.tokens)          # the last emitted token of every request
            return
        self.model.decode_step(self.batch)
        self.batch.tokens.copy_(self.batch.out_tokens)

    def warmup_and_capture(self):
        """Run the step eagerly (compiles nothing, but sets function attributes and sizes
        allocator pools), then capture it in a CUDA graph."""
        import torch
        from ..ops import _native as N

        saved = self.batch.lengths.clone()
        saved_tok = self.batch.tokens.clone()
        before = N.LAUNCHES
        self._decode_once()
        self.launches_per_step = N.LAUNCHES - before
        torch.cuda.synchronize()
        self.check()
        if self.use_graph:
            stream = torch.cuda.Stream(device=self.device)
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                self._decode_once()           # second eager run on the capture stream
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                self._decode_once()
            torch.cuda.synchronize()
        # the warm-up steps wrote KV at positions lengths..: rewind so measurements start at the prompt
        self.batch.lengths.copy_(saved)
        self.batch.tokens.copy_(saved_tok)
        if self.spec is not None:
            self.spec.emitted.zero_()
        torch.cuda.synchronize()

    def step_device(self):
        """One decode step with inputs already on the device (previous samples)."""
        if self.steps_done >= self.max_new_tokens:
            raise RuntimeError("the requests reached max_new_tokens; refill before stepping again")
        if self.graph is not None:
            self.graph.replay()
        else:
            self._decode_once()
        self.steps_done += 1
        return self.batch.out_tokens

    def step(self, host_tokens=None):
        """One decode step end to end: pinned host tokens in, pinned host samples out."""
        import torch

        src = self.host_in if host_tokens is None else host_tokens
        self.batch.tokens.copy_(src, non_blocking=True)
        self.step_device()
        self.host_out.copy_(self.batch.out_tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.host_out

    def run_replay(self, replay, cohort, *, repeat: int = 0, keys=None, steps=None):
        """Decode a RECORDED token trajectory (``tools.fixed_output.TraceTokenReplay``): every step runs the
        full model and sampler, then the recorded tokens replace the samples as the next step's inputs, so
        two cache methods (or two layouts) decode exactly the same workload.  The replay checks request
        order and sequence positions at every step.  Returns the replay's receipt."""
        import torch

        keys = list(keys) if keys is not None else [f"r{self.rank}.{i}" for i in range(self.batch.tokens.numel())]
        n = steps if steps is not None else replay.trace.data["output_tokens"]
        for _ in range(n):
            lens = self.batch.lengths[: len(keys)].tolist()
            replay.begin(cohort, repeat=repeat, keys=keys, seq_lens=lens, trace_sha256=replay.trace.sha256)
            natural = self.step_device()
            forced = replay.sample(natural)
            self.batch.tokens.copy_(forced.to(self.batch.tokens.dtype), non_blocking=True)
            replay.end()
        torch.cuda.current_stream().synchronize()
        return replay.receipt(cohort)

    def check(self):
        from ..ops import _native as N

        N.raise_on_status(self.model.status, "decode step")
        self.cache.check("decode step")

    def memory_report(self) -> dict:
        import torch

        inv = self.cache.memory_inventory()
        return {"weights_bytes": self.model.weight_bytes(), "kv_bytes": inv["device_key_value_bytes"],
                "host_kv_bytes": inv["host_key_value_bytes"], "host_records_per_rank": inv["host_record_capacity"],
                "kv_metadata_bytes": inv["metadata_bytes"], "index_bytes": self.index_pool.numel(),
                "allocated_bytes": torch.cuda.memory_allocated(self.device),
                "kv_records_per_rank": inv["device_record_capacity"]}

    def close(self):
        self.graph = None
        # the model's communication heap first (its peers' mappings are its own), then the cache's
        heap = getattr(self.model, "comm_heap", None)
        if heap is not None:
            heap.close()
            self.model.comm_heap = None
        self.cache.close()
