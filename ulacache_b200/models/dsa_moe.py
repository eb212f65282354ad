"""DeepSeek-V3.2-shaped DSA MoE decoder for decode on B200, wired to the pooled cache.

Architecture (defaults = the full model): 61 layers, hidden 7168, 128 heads; MLA with
q_lora 1536, kv_lora 512, rotary 64; a lightning indexer (64 heads x 128, top-k 2048)
per layer; 256 routed experts (top-8) + 1 shared expert with FFN dim 2048 (first
three layers dense, FFN dim 18432); vocabulary 129280; block-scaled fp8 weights
and fp8 KV records.

Per decode step and layer the data path is

    fused input projection (fp8 GEMM) -> q_b / indexer-q projection (fp8 GEMM)
    -> index key store (fp8) -> index score (fp8 tcgen05) -> radix top-k
    -> cache.prepare_sparse_attention (residency + resolve) -> cache.write (fp8 KV)
    -> fused gather + sparse MLA attention (tcgen05/TMEM) -> o_proj (fp8 GEMM)
    -> [all-reduce when tensor parallel] -> router -> grouped expert FFN (fp8 GEMM)
    -> [all-reduce]

Parallel layouts: ``tp`` (attention heads and experts sharded, queries replicated,
KV stored once and striped over ranks) and ``dpa`` (every rank decodes its own
requests with all heads against a rank-local cache; experts sharded, tokens
all-gathered around the MoE).

The reference library contains no model (it patches a serving framework); this
file is the part of that framework the cache needs in order to run stand-alone.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Optional


@dataclass(frozen=True)
class DsaMoeConfig:
    layers: int = 61
    hidden: int = 7168
    heads: int = 128
    q_lora: int = 1536
    kv_lora: int = 512
    rope_dim: int = 64
    nope_dim: int = 128
    v_dim: int = 128
    index_heads: int = 64
    index_dim: int = 128
    topk: int = 2048
    experts: int = 256
    experts_per_token: int = 8
    expert_ffn: int = 2048
    shared_experts: int = 1
    dense_layers: int = 3
    dense_ffn: int = 18432
    vocab: int = 129280
    rope_theta: float = 10000.0
    routed_scale: float = 2.5
    rms_eps: float = 1e-6
    kv_format: str = "scaled656"
    unique_layer_weights: int = 0      # 0 = every layer has its own weights
    mtp_layers: int = 0                # 1 = a multi-token-prediction draft layer (speculative decoding)

    @property
    def cache_layers(self) -> int:
        """Layers that keep KV and index entries: the decoder layers and the draft layer."""
        return self.layers + self.mtp_layers

    def __post_init__(self):
        if self.kv_lora != 512 or self.rope_dim != 64 or self.index_dim != 128 or self.index_heads != 64:
            raise ValueError("The attention and indexer kernels are built for kv_lora 512, rope 64, 64x128 indexer")
        for name in ("hidden", "q_lora", "expert_ffn", "dense_ffn"):
            if getattr(self, name) % 128:
                raise ValueError(f"{name} must be a multiple of 128 (fp8 block scaling)")
        if self.topk > 2048 or self.topk % 64:
            raise ValueError("topk must be a multiple of 64 up to 2048")

    @property
    def softmax_scale(self) -> float:
        return (self.nope_dim + self.rope_dim) ** -0.5

    def tiny(self, **kw) -> "DsaMoeConfig":
        base = dict(layers=2, hidden=512, heads=16, q_lora=256, experts=8, experts_per_token=2, expert_ffn=256,
                    dense_layers=1, dense_ffn=512, vocab=1024, topk=128)
        base.update(kw)
        return replace(self, **base)


def _rms_norm(x, weight, eps):
    import torch

    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight).to(x.dtype)


def _rope(x, cos, sin):
    """Rotate pairs (i, i + d/2) of the last dimension; cos/sin broadcast over heads."""
    import torch

    d = x.shape[-1] // 2
    a, b = x[..., :d].float(), x[..., d:].float()
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


class _Fp8Linear:
    """``y = x @ W^T`` with W stored block-scaled fp8 (Nout padded to 128)."""

    # Token rows per pass of the GEMM's ring geometry (16, 32, 64 or 128); None = the batch size.
    # A smaller value streams each weight tile once from HBM and again from L2 for every further
    # pass.  Set from ULC_DENSE_ROWS_HINT for experiments.
    rows_hint = None

    def __init__(self, nout, k, device, gen=None, std=0.02, parts=None):
        """``parts``: optional list of (rows, generator); rows of the parts add up to ``nout``
        and each part (but the last) is a multiple of 128 rows, so that replicated and
        sharded pieces of one fused weight can come from different random streams."""
        import torch
        from ..ops import fp8

        self.nout = nout
        self.pad = (nout + 127) // 128 * 128
        self.k = k
        if parts is None:
            parts = [(nout, gen)]
        qs, ss = [], []
        for i, (rows, g) in enumerate(parts):
            padded = (rows + 127) // 128 * 128
            if padded != rows and i != len(parts) - 1:
                raise ValueError("only the last part of a fused weight may need padding")
            q, sc = fp8.random_fp8_weight((padded, k), device=device, std=std, generator=g)
            qs.append(q)
            ss.append(sc)
        self.q = torch.cat(qs, dim=0) if len(qs) > 1 else qs[0]
        self.s = torch.cat(ss, dim=0) if len(ss) > 1 else ss[0]
        self.splits = fp8.pick_splits(self.pad, k)

    def nbytes(self):
        return self.q.numel() + self.s.numel() * 4

    def __call__(self, x8, sx, status=None, peer_out=None):
        from ..ops import fp8

        if peer_out is not None:
            if self.pad != self.nout:
                raise ValueError("peer outputs need an unpadded output width")
            return fp8.grouped_gemm(x8, sx, self.q, self.s, splits=self.splits, status=status, max_rows=x8.shape[0],
                                    peer_out=peer_out)
        y = fp8.grouped_gemm(x8, sx, self.q, self.s, splits=self.splits, status=status,
                             max_rows=min(self.rows_hint or x8.shape[0], x8.shape[0]))
        return y if self.pad == self.nout else y[:, : self.nout]


class _LayerWeights:
    def __init__(self, cfg: DsaMoeConfig, layer: int, *, device, attn_tp: int, tp: int, rank: int, gen=None,
                 shard_gen=None, dense_tp: Optional[int] = None, q_replicated: bool = False):
        """``gen`` draws the weights every rank must agree on (norms, input projection,
        indexer, router); ``shard_gen`` draws this rank's shard of the sharded ones.
        ``dense_tp``: shards of the dense FFN (1 = replicated, as data-parallel attention keeps it).
        ``q_replicated``: the query side of attention (q_b, W_UK) covers ALL heads on every rank while
        the output side (W_UV, o_proj) stays sharded: owner-side tensor-parallel attention."""
        import torch
        from ..ops import fp8

        c = cfg
        shard_gen = shard_gen or gen
        self.dense = layer < c.dense_layers
        heads = c.heads // attn_tp
        q_heads = c.heads if q_replicated else heads
        q_gen = gen if q_replicated else shard_gen
        bf = dict(dtype=torch.bfloat16, device=device)
        self.attn_norm = torch.ones(c.hidden, **bf)
        self.ffn_norm = torch.ones(c.hidden, **bf)
        self.q_norm = torch.ones(c.q_lora, **bf)
        self.kv_norm = torch.ones(c.kv_lora, **bf)
        # one GEMM for everything that reads the normed hidden state:
        #   q_a (q_lora) | kv_a (kv_lora + rope) | indexer key (128) | indexer head weights (64)
        self.in_splits = (c.q_lora, c.kv_lora + c.rope_dim, c.index_dim, c.index_heads)
        self.w_in = _Fp8Linear(sum(self.in_splits), c.hidden, device, gen)
        # one GEMM for everything that reads the normed q latent: q_b (heads * 192) | indexer q (64 * 128)
        self.qb_splits = (q_heads * (c.nope_dim + c.rope_dim), c.index_heads * c.index_dim)
        self.w_qb = _Fp8Linear(sum(self.qb_splits), c.q_lora, device,
                               parts=[(self.qb_splits[0], q_gen), (self.qb_splits[1], gen)])
        # absorb matrices, stored as the batched GEMM wants them (per head [N, K], K contiguous):
        # w_uk_t[h] = W_UK[h]^T maps q_nope (128) -> latent (512); w_uv_t[h] = W_UV[h]^T maps latent -> v (128)
        self.w_uk_t = (torch.randn(q_heads, c.kv_lora, c.nope_dim, device=device, generator=q_gen) * 0.05).to(torch.bfloat16)
        self.w_uv_t = (torch.randn(heads, c.v_dim, c.kv_lora, device=device, generator=shard_gen) * 0.05).to(torch.bfloat16)
        self.w_o = _Fp8Linear(c.hidden, heads * c.v_dim, device, shard_gen)
        self.index_gamma = torch.ones(c.index_dim, dtype=torch.float32, device=device)
        self.index_beta = torch.zeros(c.index_dim, dtype=torch.float32, device=device)
        if self.dense:
            dense_tp = tp if dense_tp is None else dense_tp
            ffn = c.dense_ffn // dense_tp
            dg = shard_gen if dense_tp > 1 else gen
            self.w13 = _Fp8Linear(2 * ffn, c.hidden, device, dg)
            self.w2 = _Fp8Linear(c.hidden, ffn, device, dg)
        else:
            self.local_experts = c.experts // tp
            self.expert_lo = rank * self.local_experts
            self.router = (torch.randn(c.experts, c.hidden, device=device, generator=gen) * 0.02).to(torch.bfloat16)
            self.router_bias = torch.zeros(c.experts, dtype=torch.float32, device=device)
            self.shared_fused = c.shared_experts == 1
            ne = self.local_experts + (1 if self.shared_fused else 0)
            self.e13_q, self.e13_s = fp8.random_fp8_weight((ne, 2 * c.expert_ffn, c.hidden), device=device, generator=shard_gen)
            self.e2_q, self.e2_s = fp8.random_fp8_weight((ne, c.hidden, c.expert_ffn), device=device, generator=shard_gen)
            # One shared expert has the shape of a routed one: every rank keeps a whole copy as
            # local expert number `local_experts` and runs it, inside the same grouped GEMM, on its
            # own slice of the tokens.  Other counts run as a separate FFN sharded over the ranks.
            if self.shared_fused:
                # (the copy every rank keeps must be the same: drawn from the common stream)
                q13, s13 = fp8.random_fp8_weight((1, 2 * c.expert_ffn, c.hidden), device=device, generator=gen)
                q2, s2 = fp8.random_fp8_weight((1, c.hidden, c.expert_ffn), device=device, generator=gen)
                self.e13_q[-1].copy_(q13[0]); self.e13_s[-1].copy_(s13[0])
                self.e2_q[-1].copy_(q2[0]); self.e2_s[-1].copy_(s2[0])
            elif c.shared_experts > 1:
                sf = c.shared_experts * c.expert_ffn // tp
                self.s13 = _Fp8Linear(2 * sf, c.hidden, device, shard_gen)
                self.s2 = _Fp8Linear(c.hidden, sf, device, shard_gen)

    def shard_(self, cfg: DsaMoeConfig, *, tp: int, rank: int, attn_tp: int, dense_tp: int, q_replicated: bool):
        """Turn FULL (one-rank) weights into this rank's shard in place, so that an N-rank model and a
        one-rank model built from the same random stream are the same network (validation runs on
        small configurations; the full-size model draws each rank's shard directly)."""
        import torch

        c = cfg

        def rows(lin, lo, hi):                    # keep output rows [lo, hi) (multiples of 128)
            lin.q = lin.q[lo // 128: hi // 128].contiguous()
            lin.s = lin.s[lo // 128: hi // 128].contiguous()
            lin.nout = lin.pad = hi - lo

        def cols(lin, lo, hi):                    # keep input columns [lo, hi) (multiples of 128)
            lin.q = lin.q[:, lo // 128: hi // 128].contiguous()
            lin.s = lin.s[:, lo // 128: hi // 128].contiguous()
            lin.k = hi - lo

        if attn_tp > 1:
            heads = c.heads // attn_tp
            h0 = rank * heads
            if not q_replicated:
                per = c.nope_dim + c.rope_dim
                keep = torch.cat([self.w_qb.q[h0 * per // 128:(h0 + heads) * per // 128],
                                  self.w_qb.q[c.heads * per // 128:]])
                keep_s = torch.cat([self.w_qb.s[h0 * per // 128:(h0 + heads) * per // 128],
                                    self.w_qb.s[c.heads * per // 128:]])
                self.w_qb.q, self.w_qb.s = keep.contiguous(), keep_s.contiguous()
                self.qb_splits = (heads * per, c.index_heads * c.index_dim)
                self.w_qb.nout = self.w_qb.pad = sum(self.qb_splits)
                self.w_uk_t = self.w_uk_t[h0:h0 + heads].contiguous()
            self.w_uv_t = self.w_uv_t[h0:h0 + heads].contiguous()
            cols(self.w_o, h0 * c.v_dim, (h0 + heads) * c.v_dim)
        from ..ops import fp8

        for lin in (self.w_qb, self.w_o):
            lin.splits = fp8.pick_splits(lin.pad, lin.k)
        if self.dense:
            if dense_tp > 1:
                ffn = c.dense_ffn // dense_tp
                f0 = rank * ffn
                q, sc = self.w13.q, self.w13.s
                self.w13.q = torch.cat([q[f0 // 128:(f0 + ffn) // 128],
                                        q[(c.dense_ffn + f0) // 128:(c.dense_ffn + f0 + ffn) // 128]]).contiguous()
                self.w13.s = torch.cat([sc[f0 // 128:(f0 + ffn) // 128],
                                        sc[(c.dense_ffn + f0) // 128:(c.dense_ffn + f0 + ffn) // 128]]).contiguous()
                self.w13.nout = self.w13.pad = 2 * ffn
                cols(self.w2, f0, f0 + ffn)
                for lin in (self.w13, self.w2):
                    lin.splits = fp8.pick_splits(lin.pad, lin.k)
        elif tp > 1:
            local = c.experts // tp
            lo = rank * local
            pick = list(range(lo, lo + local)) + ([c.experts] if self.shared_fused else [])
            idx = torch.tensor(pick, device=self.e13_q.device)
            self.e13_q, self.e13_s = self.e13_q[idx].contiguous(), self.e13_s[idx].contiguous()
            self.e2_q, self.e2_s = self.e2_q[idx].contiguous(), self.e2_s[idx].contiguous()
            self.local_experts, self.expert_lo = local, lo

    def nbytes(self) -> int:
        import torch

        n = 0
        for v in vars(self).values():
            if torch.is_tensor(v):
                n += v.numel() * v.element_size()
            elif isinstance(v, _Fp8Linear):
                n += v.nbytes()
        return n


@dataclass
class DecodeBatch:
    """Device-resident state of the running requests (graph-replay safe: every step
    only mutates these tensors in place)."""

    tokens: object            # int32 [B] current input token of each request
    lengths: object           # int32 [B] tokens already in the cache (position of the new token)
    req_pages: object         # int32 [B, max_alloc_pages] allocation page of each 64*ranks-token stretch
    out_tokens: object        # int32 [B] sampled tokens of the last step


@dataclass
class SpeculativeBatch:
    """Device state of speculative decoding (graph-replay safe)."""

    tokens: object            # int32 [B] input token of each request (the last emitted one)
    lengths: object           # int32 [B] tokens in the cache = position of the input token
    req_pages: object         # int32 [B, pages]
    drafts: object            # int32 [B, S] draft tokens for the next S positions
    out: object               # int32 [B, S + 1] the model's tokens of the last step (first accepted + 1 are valid)
    accepted: object          # int32 [B] accepted draft tokens of the last step
    emitted: object           # int64 [1] tokens emitted so far (sum of accepted + 1)


class DsaMoeModel:
    def __init__(self, cfg: DsaMoeConfig, *, device, cache, index_pool, tp: int = 1, rank: int = 0,
                 group=None, cpu_group=None, mode: str = "tp", max_batch: int = 64, max_context: int = 65536,
                 seed: int = 0, comm: str = "peer", deterministic: Optional[bool] = None,
                 tp_attention: str = "owner", weights_from_full: bool = False, kv_layout: str = "pooled"):
        import torch
        from ..ops import _native as N
        from ..ops import records

        if kv_layout not in ("pooled", "replicated"):
            raise ValueError("kv_layout must be pooled or replicated")
        if mode not in ("tp", "dpa"):
            raise ValueError("mode must be tp or dpa")
        if cfg.heads % tp or cfg.experts % tp:
            raise ValueError("heads and experts must divide by the parallel degree")
        self.cfg, self.device, self.cache, self.tp, self.rank, self.group, self.mode = cfg, torch.device(device), cache, tp, rank, group, mode
        # The radix select emits its winners in no particular order, so attention sums them in an
        # order that varies from run to run (results agree to fp32 rounding, not bit for bit).
        # ``deterministic`` sorts every selection first: bit-reproducible steps for tests and debugging.
        import os as _os

        self.deterministic = (_os.environ.get("ULC_DETERMINISTIC", "0") == "1") if deterministic is None else deterministic
        self.shared_placement = _os.environ.get("ULC_MOE_SHARED_PLACEMENT", "0") == "1"
        # W_UV product with the o_proj input quantiser in its epilogue: one launch fewer, but measured
        # slower than the two kernels at 32 rows (two TMEM passes in the epilogue), so off by default
        self._fused_oquant = _os.environ.get("ULC_FUSED_OQUANT", "0") == "1"
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 0
        hint = _os.environ.get("ULC_DENSE_ROWS_HINT", "")
        if hint:
            _Fp8Linear.rows_hint = int(hint)
        self.attn_tp = tp if mode == "tp" else 1          # heads are sharded only in tp mode
        # owners of the striped pool.  ``kv_layout="replicated"`` is the baseline a pooled cache is measured
        # against: tensor-parallel heads, but every rank keeps (and writes) ALL records and index keys, so
        # attention and the indexer are rank-local and the KV capacity is that of one GPU
        self.kv_ranks = tp if (mode == "tp" and kv_layout == "pooled") else 1
        self.kv_rank = rank if self.kv_ranks > 1 else 0
        self.dpa = mode == "dpa" and tp > 1               # tokens gathered / scattered around the experts
        # tensor-parallel attention over the striped pool: "gather" = every rank reads all selected
        # records (peers' pools included) for its own heads; "owner" = every rank attends over the
        # records it owns for all heads and the partial results are exchanged by head
        if tp_attention not in ("owner", "gather"):
            raise ValueError("tp_attention must be owner or gather")
        self.owner_attention = (mode == "tp" and tp > 1 and tp_attention == "owner" and comm == "peer"
                                and self.device.type == "cuda" and self.kv_ranks > 1)
        self.max_batch, self.max_context = max_batch, max_context
        gen = torch.Generator(device=self.device).manual_seed(seed)
        shard_gen = torch.Generator(device=self.device).manual_seed(seed + 7919 * (rank + 1))
        self.status = N.new_status(self.device)
        unique = cfg.unique_layer_weights or cfg.layers
        self._unique = []
        self.weights_from_full = weights_from_full
        for l in range(min(unique, cfg.layers)):
            # unique set l is dense when l < dense_layers; MoE layers cycle over the MoE sets
            if weights_from_full:
                # (validation) the one-rank network from the common stream, cut down to this rank's shard
                w = _LayerWeights(cfg, l, device=self.device, attn_tp=1, tp=1, rank=0, gen=gen, shard_gen=gen, dense_tp=1)
                w.shard_(cfg, tp=tp, rank=rank, attn_tp=self.attn_tp, dense_tp=1 if self.dpa else tp,
                         q_replicated=self.owner_attention)
                self._unique.append(w)
                continue
            self._unique.append(_LayerWeights(cfg, l, device=self.device, attn_tp=self.attn_tp, tp=tp, rank=rank,
                                              gen=gen, shard_gen=shard_gen, dense_tp=1 if self.dpa else tp,
                                              q_replicated=self.owner_attention))
        self.embed = (torch.randn(cfg.vocab, cfg.hidden, device=self.device, generator=gen) * 0.02).to(torch.bfloat16)
        self.final_norm = torch.ones(cfg.hidden, dtype=torch.bfloat16, device=self.device)
        self.vocab_local = (cfg.vocab + tp - 1) // tp
        if weights_from_full and tp > 1:
            if cfg.vocab % (128 * tp):
                raise ValueError("weights_from_full needs a vocabulary that splits into 128-row tiles per rank")
            full = _Fp8Linear(cfg.vocab, cfg.hidden, self.device, gen)
            full.q = full.q[rank * self.vocab_local // 128:(rank + 1) * self.vocab_local // 128].contiguous()
            full.s = full.s[rank * self.vocab_local // 128:(rank + 1) * self.vocab_local // 128].contiguous()
            full.nout = full.pad = self.vocab_local
            self.lm_head = full
        else:
            self.lm_head = _Fp8Linear(self.vocab_local, cfg.hidden, self.device, gen if weights_from_full else shard_gen)
        # rotary tables
        half = cfg.rope_dim // 2
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, device=self.device).float() / half))
        ang = torch.arange(max_context, device=self.device).float()[:, None] * inv[None, :]
        self.cos, self.sin = torch.cos(ang), torch.sin(ang)
        self.cos_sin = torch.cat([self.cos, self.sin], dim=1).contiguous()       # [pos, 64] for the index-key kernel
        self.index_pool = index_pool                                              # uint8 [layers, pages, 8448]
        self.index_views = [records.make_index_view(page_ptrs=[index_pool[l].data_ptr()] * max(self.kv_ranks, 1),
                                                    pages_per_rank=index_pool.shape[1], ranks=self.kv_ranks,
                                                    my_rank=self.kv_rank)
                            for l in range(cfg.cache_layers)]
        # multi-token-prediction draft: h' = W [norm(emb(next token)); norm(h)] -> one decoder layer -> shared head
        self.mtp = None
        if cfg.mtp_layers:
            if cfg.mtp_layers != 1:
                raise ValueError("one draft layer is supported")
            self.mtp = dict(enorm=torch.ones(cfg.hidden, dtype=torch.bfloat16, device=self.device),
                            hnorm=torch.ones(cfg.hidden, dtype=torch.bfloat16, device=self.device),
                            proj=_Fp8Linear(cfg.hidden, 2 * cfg.hidden, self.device, gen),
                            layer=_LayerWeights(cfg, cfg.dense_layers, device=self.device, attn_tp=self.attn_tp, tp=tp,
                                                rank=rank, gen=gen, shard_gen=shard_gen, dense_tp=1 if self.dpa else tp,
                                                q_replicated=self.owner_attention))
        self._ag_by_rows = {}
        # The index-score kernel leaves each row's score histogram in this workspace and the radix
        # select starts from it (ULC_TOPK_FUSED=0: separate score and select kernels, for comparison).
        self._topk_ws = None
        self._topk_rows = _os.environ.get("ULC_TOPK_ROWS", "1") == "1"      # (0: the histogram pair at every row count)
        if self.device.type == "cuda" and _os.environ.get("ULC_TOPK_FUSED", "1") == "1":
            from ..ops import topk as _topk

            self._topk_ws = _topk.workspace(max_batch, self.device)
        self._nvtx = _os.environ.get("ULC_NVTX", "0") == "1"
        self._nvtx_open = False
        self.record_selections = None       # a list here makes every layer append its selected record IDs
        self.record_current = None          # ... and the ids of the records the step is writing (one per row)
        self.record_sublayers = None        # ... and (attention output, feed-forward output) of every layer
        self.record_routing = None          # ... and (expert choice, gate) of every MoE layer
        self.force_routing = None           # a list of (choice, gate) here replaces the router's decision, one
        #                                     entry per MoE layer in order (eager runs only: two layouts of one
        #                                     network compared without near-tied experts flipping between them)
        self.last_logits = None
        if self.deterministic:
            # split-K sums partial products with fp32 atomics, in an order that varies from run to run
            layers = list(self._unique) + ([self.mtp["layer"]] if self.mtp else [])
            linears = [v for w in layers for v in vars(w).values() if isinstance(v, _Fp8Linear)] + [self.lm_head]
            if self.mtp:
                linears.append(self.mtp["proj"])
            for lin in linears:
                lin.splits = 1
        # cross-rank reductions and the candidate exchange go through peer memory unless asked otherwise
        self.comm = comm if (tp > 1 and self.device.type == "cuda") else "none"
        self.ar = self.cand = self.comm_heap = None
        if self.comm == "peer":
            from ..parallel.peer_collectives import PeerAllReduce, PeerCandidateExchange
            from ..parallel.symmetric import SymmetricHeap

            need = 2 * tp * max_batch * cfg.hidden * 2 + (4 << 20)
            need += 4 * tp * max_batch * cfg.topk * 4 if mode == "tp" else 4 * tp * max_batch * (cfg.hidden + 1024)
            if self.owner_attention:
                need += 2 * max_batch * cfg.heads * (512 * 2 + 4) + (1 << 20)
            need *= 2 if cfg.mtp_layers else 1          # the draft passes gather other row counts
            self.comm_heap = SymmetricHeap(cpu_group=cpu_group, rank=rank, world_size=tp, nbytes=need,
                                           device=self.device)
            self.ar = PeerAllReduce(self.comm_heap, max_batch, cfg.hidden)
            if mode == "tp":
                self.cand = PeerCandidateExchange(self.comm_heap, max_batch, cfg.topk)
                if self.owner_attention:
                    from ..parallel.peer_collectives import PeerHeadExchange

                    self.head_x = PeerHeadExchange(self.comm_heap, max_batch, cfg.heads)
                    if hasattr(cache, "declare_local_readers_only"):
                        cache.declare_local_readers_only()
            else:
                from ..parallel.peer_collectives import PeerAllGather

                act = [(cfg.hidden, torch.uint8), (cfg.hidden // 128, torch.float32)]
                route = [(cfg.experts_per_token, torch.int32), (cfg.experts_per_token, torch.float32)]
                self.ag_moe = PeerAllGather(self.comm_heap, max_batch, act + route, name="ag_moe")
                self.ag_head = PeerAllGather(self.comm_heap, max_batch, act, name="ag_head")

    # ---------------------------------------------------------------- helpers --
    def enable_profile(self, on: bool = True):
        """Per-section CUDA-event timers (eager mode only); read them with ``profile_summary``."""
        self._prof = {} if on else None

    def _mark(self, name: str):
        """Close the running section and open ``name``: a CUDA-event section when profiling, and an
        NVTX range when ``ULC_NVTX=1`` (ranges nest under the step's range and show up in any
        NVTX-aware timeline; they are recorded during graph capture only as host markers)."""
        if self._nvtx:
            import torch

            if self._nvtx_open:
                torch.cuda.nvtx.range_pop()
            self._nvtx_open = name != "end"              # "end" closes the step's last section
            if self._nvtx_open:
                torch.cuda.nvtx.range_push(name)
        prof = getattr(self, "_prof", None)
        if prof is None:
            return
        import torch

        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        prof.setdefault("__events__", []).append((name, ev))

    def profile_summary(self) -> dict:
        import torch

        torch.cuda.synchronize()
        evs = (self._prof or {}).get("__events__", [])
        out = {}
        for (name, a), (_, b) in zip(evs, evs[1:]):
            if name != "end":
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return dict(sorted(out.items(), key=lambda kv: -kv[1]))

    def layer_weights(self, layer: int) -> _LayerWeights:
        c = self.cfg
        if len(self._unique) >= c.layers:
            return self._unique[layer]
        if layer < c.dense_layers:
            return self._unique[layer % max(1, min(c.dense_layers, len(self._unique)))]
        moe = [w for w in self._unique if not w.dense]
        return moe[(layer - c.dense_layers) % len(moe)]

    def weight_bytes(self) -> int:
        return sum(w.nbytes() for w in self._unique) + self.embed.numel() * 2 + self.lm_head.nbytes()

    def _all_reduce(self, t):
        """Library all-reduce (the baseline path).  Returns a (tensor, slots, stride) delta."""
        if self.tp > 1:
            import torch.distributed as dist

            dist.all_reduce(t, group=self.group)
        return (t.contiguous(), 1, 0)

    def _gather_rows(self, tensors, ag):
        """All-gather row blocks over the ranks (data-parallel attention): peer stores, or the
        library collective on the baseline path."""
        if self.comm == "peer":
            rows = tensors[0].shape[0]
            if rows != ag.rows:
                # another row count (draft / verify passes): its own receive buffers, created on first
                # use (every rank runs the same sequence, so heap offsets agree)
                key = (id(ag), rows)
                if key not in self._ag_by_rows:
                    from ..parallel.peer_collectives import PeerAllGather

                    self._ag_by_rows[key] = PeerAllGather(self.comm_heap, rows, ag.widths, name=f"ag{len(self._ag_by_rows)}_{rows}")
                ag = self._ag_by_rows[key]
            return ag.gather([t.contiguous() for t in tensors])
        import torch
        import torch.distributed as dist

        out = []
        for t in tensors:
            t = t.contiguous()
            g = torch.empty((self.tp * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(g, t, group=self.group)
            out.append(g)
        return out

    def _peer_targets(self):
        """Receive-slot addresses for a producer kernel, or None when the library path is used."""
        return self.ar.targets() if self.ar is not None else None

    def _peer_finish(self):
        return self.ar.finish()

    def _quant(self, x):
        from ..ops import fp8

        return fp8.act_quant(x.contiguous())

    def new_token_ids(self, batch: DecodeBatch):
        """Logical record ID of the token each request writes this step."""
        import torch

        span = 64 * self.kv_ranks
        pos = batch.lengths.long()
        page = torch.gather(batch.req_pages.long(), 1, (pos // span).unsqueeze(1)).squeeze(1)
        return (page * span + pos % span).to(torch.int32)

    # ------------------------------------------------------------------ layers --
    def _attention(self, layer: int, w: _LayerWeights, h8, hs, batch: DecodeBatch, new_ids):
        """Attention sub-layer on the normed, quantised hidden state; returns its output
        (already summed over tensor-parallel ranks), to be added to the residual."""
        import torch
        from ..cache.access import SparseAttentionAccessPlan
        from ..ops import fp8, gemm, glue, indexer, records, sparse_mla

        c = self.cfg
        B = h8.shape[0]
        out_heads = c.heads // self.attn_tp                       # heads of W_UV / o_proj on this rank
        heads = c.heads if self.owner_attention else out_heads    # heads of the query side
        self._mark("attn.w_in gemm")
        fused = w.w_in(h8, hs, self.status)
        self._mark("attn.prep kernels")
        q8, qs, latent, k_rope = glue.mla_prep(fused, c.q_lora, w.q_norm, w.kv_norm, c.rms_eps, self.cos_sin,
                                               batch.lengths)
        self._mark("attn.w_qb gemm")
        qb = w.w_qb(q8, qs, self.status)
        self._mark("attn.prep kernels")
        ik_off = c.q_lora + c.kv_lora + c.rope_dim
        _, q_rope, iq8, iwf = glue.q_prep(qb, heads, self.cos_sin, batch.lengths, fused, ik_off + c.index_dim,
                                          c.index_heads ** -0.5, want_nope_t=False)
        self._mark("attn.absorb gemm")
        # q_lat[b, h, :] = q_nope[b, h, :] @ W_UK[h], read in place from the projection output
        q_nope = torch.as_strided(qb, (B, heads, c.nope_dim), (qb.stride(0), c.nope_dim + c.rope_dim, 1))
        if gemm.many_rows(B):     # prefill-sized: head-major storage, which the library's batched product writes in place
            q_lat = torch.empty((heads, B, c.kv_lora), dtype=torch.bfloat16, device=qb.device).transpose(0, 1)
        else:
            q_lat = torch.empty((B, heads, c.kv_lora), dtype=torch.bfloat16, device=qb.device)
        gemm.batched_linear(q_nope, w.w_uk_t, q_lat)

        # ---- indexer: store this token's key, score the context, take the top-k
        self._mark("index.key store")
        records.index_key_store(self.index_views[layer], fused[:, ik_off:ik_off + c.index_dim], new_ids,
                                gamma=w.index_gamma, beta=w.index_beta, cos_sin=self.cos_sin,
                                positions=batch.lengths, owner_only=True, status=self.status)
        self._mark("index.score")
        # prefill-sized row counts: plain scores, then the row-parallel select with explicit lengths (the histogram
        # epilogue and the select that starts from it are built for a few dozen rows)
        many = self._topk_rows and B >= 48 and self.kv_ranks == 1
        ws = None if many else self._topk_ws
        logits = indexer.index_score(iq8, iwf, batch.req_pages, self._ctx, self.index_pool[layer],
                                     ranks=self.kv_ranks, rank=self.kv_rank,
                                     status=self.status, topk_workspace=ws)
        self._mark("index.topk")
        sel = self._select(logits, batch, ws, self._ctx if many else None)
        if self.deterministic:
            sel = torch.sort(sel, dim=1, descending=True).values.contiguous()
        if self.record_selections is not None:
            self.record_selections.append(sel.clone())          # (eager runs only: for oracles and traces)
        if self.record_current is not None:
            self.record_current.append(new_ids.clone())

        # ---- cache: residency + resolve, publish the new KV, attend
        self._mark("cache.plan+write")
        self.cache.prepare_sparse_attention(layer, SparseAttentionAccessPlan(sel, new_ids))
        self.cache.write(new_ids, layer, (latent, k_rope))
        view = self.cache.get_resident_attention_inputs(layer)
        self._mark("attn.sparse_mla")
        fmt = 0 if c.kv_format == "scaled656" else 2
        if self.owner_attention:
            from ..parallel.peer_collectives import owner_localize

            mine, counts = owner_localize(view.device_record_indices, self.rank)
            o_part, lse_part = sparse_mla.sparse_mla_decode_strided_auto(
                view.pool_view, q_lat, q_rope, mine, c.softmax_scale, fmt_code=fmt, lens=counts, status=self.status)
            self._mark("comm")
            o_lat = self.head_x.exchange_and_merge(o_part, lse_part)
        else:
            o_lat, _ = sparse_mla.sparse_mla_decode_strided_auto(
                view.pool_view, q_lat, q_rope, view.device_record_indices, c.softmax_scale, fmt_code=fmt,
                status=self.status)
        self.cache.finish_layer_attention(layer)
        self._mark("attn.absorb gemm")
        # o[b, h, :] = o_lat[b, h, :] @ W_UV[h]; each head's 128 values are one fp8 group of the o_proj
        # input, so the product leaves its kernel quantised
        if self._fused_oquant:
            o8, os_ = gemm.batched_linear_quant(o_lat, w.w_uv_t, status=self.status)
        else:                                   # separate product and quantiser (ULC_FUSED_OQUANT=0, for comparison)
            o = torch.empty((B, out_heads * c.v_dim), dtype=torch.bfloat16, device=qb.device)
            gemm.batched_linear(o_lat, w.w_uv_t, o.view(B, out_heads, c.v_dim))
            o8, os_ = fp8.act_quant(o)
        self._mark("attn.w_o gemm")
        if self.attn_tp > 1 and self.ar is not None:
            w.w_o(o8, os_, self.status, peer_out=self._peer_targets())      # scatter phase in the GEMM epilogue
            self._mark("comm")
            return self._peer_finish()
        out = w.w_o(o8, os_, self.status)
        self._mark("comm")
        return self._all_reduce(out) if self.attn_tp > 1 else (out, 1, 0)

    def _select(self, logits, batch: DecodeBatch, hist_workspace=None, lengths=None):
        """Top-k over the (local shard of the) scores -> logical IDs [B, topk]."""
        from ..ops import indexer

        c = self.cfg
        if self.kv_ranks == 1:
            return indexer.select_topk(logits, c.topk, batch.req_pages, n_q=1, hist_workspace=hist_workspace, lengths=lengths)
        return self._distributed_select(logits, batch)

    def _distributed_select(self, logits, batch: DecodeBatch):
        """Each rank takes its local top-k, candidates are exchanged, every rank merges
        the ranks * k candidates (all ranks end with the same selection)."""
        import torch
        import torch.distributed as dist
        from ..ops import indexer, topk as topk_op

        c = self.cfg
        ids, vals = indexer.select_topk(logits, c.topk, batch.req_pages, n_q=1, ranks=self.kv_ranks, rank=self.rank,
                                        with_values=True, hist_workspace=self._topk_ws)
        if self.cand is not None:
            cand_v, cand_i = self.cand.exchange(ids, vals)
            return topk_op.topk(cand_v, c.topk, in_idx=cand_i)
        all_ids = torch.empty((self.tp,) + ids.shape, dtype=ids.dtype, device=ids.device)
        all_vals = torch.empty((self.tp,) + vals.shape, dtype=vals.dtype, device=vals.device)
        dist.all_gather_into_tensor(all_ids, ids, group=self.group)
        dist.all_gather_into_tensor(all_vals, vals, group=self.group)
        cand_v = all_vals.permute(1, 0, 2).reshape(ids.shape[0], -1).contiguous()
        cand_i = all_ids.permute(1, 0, 2).reshape(ids.shape[0], -1).contiguous()
        return topk_op.topk(cand_v, c.topk, in_idx=cand_i)

    def _ffn(self, w: _LayerWeights, h, h8, hs):
        """Feed-forward sub-layer on the normed hidden state (bf16 ``h`` for the router, fp8 for
        the GEMMs); returns its output summed over ranks."""
        import torch
        from ..ops import fp8, gemm, glue

        c = self.cfg
        B = h8.shape[0]
        if w.dense:
            self._mark("ffn.dense gemms")
            mid = w.w13(h8, hs, self.status)
            m8, ms = fp8.act_quant(mid, swiglu=True)
            if self.dpa:
                return (w.w2(m8, ms, self.status), 1, 0)           # replicated: nothing to reduce
            if self.tp > 1 and self.ar is not None:
                w.w2(m8, ms, self.status, peer_out=self._peer_targets())
                self._mark("comm")
                return self._peer_finish()
            out = w.w2(m8, ms, self.status)
            self._mark("comm")
            return self._all_reduce(out)
        self._mark("moe.route+permute")
        # router scores on the same tcgen05 GEMM as the absorb products (split-K sums with atomics:
        # one split when bit-reproducible steps are asked for)
        logits = gemm.linear(h, w.router, splits=1 if self.deterministic else 0, status=self.status)
        choice, gate = glue.moe_topk(logits, w.router_bias, c.experts_per_token, c.routed_scale)
        if self.force_routing is not None:
            choice, gate = self.force_routing.pop(0)
        if self.record_routing is not None:             # (eager runs only: for oracles)
            self.record_routing.append((choice.clone(), gate.clone()))
        b_local = B
        if self.dpa:
            # every rank's experts see every rank's tokens: gather activations and routing decisions
            self._mark("comm")
            h8, hs, choice, gate = self._gather_rows([h8, hs, choice, gate], getattr(self, "ag_moe", None))
            B = h8.shape[0]
            self._mark("moe.route+permute")
        shared_rows = None
        if w.shared_fused:
            per = (B + self.tp - 1) // self.tp            # this rank's slice of the tokens
            s_lo = min(B, self.rank * per)
            shared_rows = (s_lo, max(0, min(per, B - s_lo)))
        placement = None
        if self.shared_placement and w.shared_fused:
            # experimental: start the shared expert's (longer) items on CTAs that get no extra item
            placement = (w.e13_q.shape[1], w.e2_q.shape[1])
        route = glue.moe_sort(choice, gate, w.expert_lo, w.local_experts, shared_rows=shared_rows,
                              gemm_tiles=placement, grid=self._sm_count if placement else 0)
        x8p, xsp = glue.moe_gather(h8, hs, route)
        # expected rows per expert decide the kernel's ring geometry (any value is correct)
        # (the shared expert's slice may be longer: it then takes several passes over its tiles)
        # The 16-token geometry streams weights fastest; an expert with more rows just takes another
        # pass over its tiles (from L2), which is rare while the mean stays well below 16.
        avg = B * c.experts_per_token / c.experts
        hint = 16 if avg <= 10 else 32 if avg <= 24 else 64 if avg <= 50 else 128
        hint = min(hint, max(16, B))
        self._mark("moe.w13 grouped gemm")
        mid = fp8.grouped_gemm(x8p, xsp, w.e13_q, w.e13_s, route["offs"], status=self.status, max_rows=hint,
                               active=route["active"])
        self._mark("moe.swiglu quant")
        # `mid` is sized for every (token, choice) pair; only the rows routed to this rank's experts exist
        m8, ms = fp8.act_quant(mid, swiglu=True, row_limit=route["offs"][route["experts"]:])
        self._mark("moe.w2 grouped gemm")
        y = fp8.grouped_gemm(m8, ms, w.e2_q, w.e2_s, route["offs"], status=self.status, max_rows=hint,
                             active=route["active2"])
        shared = None
        if not w.shared_fused and c.shared_experts > 0:
            self._mark("moe.shared expert")
            smid = w.s13(h8, hs, self.status)
            s8, ss = fp8.act_quant(smid, swiglu=True)
            shared = w.s2(s8, ss, self.status)
        self._mark("moe.combine")
        if self.tp > 1 and self.ar is not None:
            # all-reduce (tp) or reduce-scatter back to the rank that owns each token (dpa)
            glue.moe_combine(y, route, shared, B, c.hidden, peer_out=self._peer_targets(),
                             rows_per_peer=b_local if self.dpa else 0)
            self._mark("comm")
            return self._peer_finish()
        out = glue.moe_combine(y, route, shared, B, c.hidden)
        self._mark("comm")
        if self.dpa:
            import torch.distributed as dist

            mine = torch.empty((b_local, c.hidden), dtype=out.dtype, device=out.device)
            dist.reduce_scatter_tensor(mine, out, group=self.group)
            return (mine, 1, 0)
        return self._all_reduce(out)

    def _layer(self, layer: int, w: _LayerWeights, x, delta, batch: DecodeBatch, new_ids):
        """One decoder layer on the residual stream ``x`` (updated in place by the fused norms);
        ``delta`` is what the previous sub-layer left to be added.  Returns this layer's delta."""
        from ..ops import glue

        c = self.cfg
        self._mark("norm+quant")
        _, h8, hs = glue.add_rmsnorm_quant(x, delta[0], w.attn_norm, c.rms_eps, n_slots=delta[1], slot_stride=delta[2])
        attn = self._attention(layer, w, h8, hs, batch, new_ids)
        self._mark("norm+quant")
        h, h8, hs = glue.add_rmsnorm_quant(x, attn[0], w.ffn_norm, c.rms_eps, want_h=not w.dense,
                                           n_slots=attn[1], slot_stride=attn[2])
        out = self._ffn(w, h, h8, hs)
        if self.record_sublayers is not None:           # (eager single-rank runs only: for oracles)
            self.record_sublayers.append((attn[0].clone(), out[0].clone()))
        return out

    def _head(self, x, delta, n_rows):
        """Final norm, sharded lm_head, greedy sample -> int32 [n_rows] (this rank's rows)."""
        import torch
        from ..ops import glue

        c = self.cfg
        _, h8, hs = glue.add_rmsnorm_quant(x, delta[0], self.final_norm, c.rms_eps, n_slots=delta[1], slot_stride=delta[2])
        if self.dpa:
            h8, hs = self._gather_rows([h8, hs], getattr(self, "ag_head", None))    # vocabulary is sharded
        logits = self.lm_head(h8, hs, self.status).float()
        self.last_logits = logits                               # this rank's vocabulary shard, fp32
        val, idx = logits.max(dim=-1)
        idx = idx + self.rank * self.vocab_local if self.tp > 1 else idx
        if self.tp > 1:
            import torch.distributed as dist

            vals = torch.empty((self.tp, val.numel()), dtype=val.dtype, device=val.device)
            idxs = torch.empty((self.tp, idx.numel()), dtype=idx.dtype, device=idx.device)
            dist.all_gather_into_tensor(vals, val, group=self.group)
            dist.all_gather_into_tensor(idxs, idx, group=self.group)
            idx = torch.gather(idxs, 0, vals.argmax(dim=0, keepdim=True)).squeeze(0)
            if self.dpa:
                idx = idx[self.rank * n_rows:(self.rank + 1) * n_rows]
        return idx.clamp(max=c.vocab - 1).to(torch.int32)

    def mtp_step(self, batch: DecodeBatch, hidden, next_tokens):
        """Draft layer: consumes the main model's (or its own previous) hidden state of each row and
        the token that FOLLOWS that row's position; writes the draft layer's KV / index entry at the
        row's position; returns (draft of the token after ``next_tokens``, new hidden)."""
        import torch
        from ..ops import fp8

        c, m = self.cfg, self.mtp
        self.cache.begin_model_forward()
        e = self.embed[next_tokens.long()]
        xin = torch.cat([_rms_norm(e, m["enorm"], c.rms_eps), _rms_norm(hidden, m["hnorm"], c.rms_eps)], dim=-1)
        x8, xs = fp8.act_quant(xin.contiguous())
        x = m["proj"](x8, xs, self.status).contiguous()
        new_ids = self.new_token_ids(batch)
        self._ctx = batch.lengths + 1
        delta = self._layer(c.layers, m["layer"], x, (None, 1, 0), batch, new_ids)
        self.cache.finish_model_forward()
        tok = self._head(x, delta, batch.tokens.shape[0])
        return tok, x

    def speculative_step(self, st: "SpeculativeBatch", force_accept: Optional[int] = None):
        """One linear-chain speculative decode step (draft length S = ``st.drafts.shape[1]``).

        Verify: the main model runs on S + 1 rows per request - the input token and the S draft
        tokens, at consecutive positions (rows of one request see one another causally because every
        row's KV is written before any row attends).  Accept the longest draft prefix that matches
        the model's own greedy tokens, emit those plus one bonus token.  Draft: the draft layer runs
        over the same rows (which also rebuilds its KV for the accepted positions), its prediction
        behind the last accepted row starts the next chain, S - 1 more single-row draft steps
        extend it.  KV written for rejected positions is overwritten by the next step.
        ``force_accept``: use this accepted length instead of the comparison (throughput studies at
        a given acceptance, as a fixed-trajectory replay would give)."""
        import torch

        B, S = st.drafts.shape
        R = B * (S + 1)
        dev = st.tokens.device
        steps = torch.arange(S + 1, device=dev, dtype=torch.int32)
        rows_tok = torch.cat([st.tokens.unsqueeze(1), st.drafts], dim=1).reshape(-1).contiguous()
        rows_len = (st.lengths.unsqueeze(1) + steps).reshape(-1).contiguous()
        rows_pages = st.req_pages.repeat_interleave(S + 1, dim=0).contiguous()
        vb = DecodeBatch(tokens=rows_tok, lengths=rows_len.clone(), req_pages=rows_pages,
                         out_tokens=torch.zeros(R, dtype=torch.int32, device=dev))
        self.decode_step(vb)
        y = vb.out_tokens.view(B, S + 1)
        hidden = self.last_hidden                                                  # [R, hidden]
        if force_accept is None:
            acc = (st.drafts == y[:, :S]).to(torch.int32).cumprod(dim=1).sum(dim=1).to(torch.int32)
        else:
            acc = torch.full((B,), min(int(force_accept), S), dtype=torch.int32, device=dev)
        st.out.copy_(y)
        st.accepted.copy_(acc)
        st.emitted.add_((acc + 1).sum())
        new_tok = torch.gather(y, 1, acc.long().unsqueeze(1)).squeeze(1)
        # draft pass over the verify rows: (hidden of position q, token of position q + 1)
        mb = DecodeBatch(tokens=rows_tok, lengths=rows_len.clone(), req_pages=rows_pages, out_tokens=vb.out_tokens)
        e, hm = self.mtp_step(mb, hidden, y.reshape(-1))
        pick = (torch.arange(B, device=dev) * (S + 1) + acc.long())
        d = e[pick]
        h_prev = hm[pick].contiguous()
        st.lengths.add_(acc + 1)
        st.tokens.copy_(new_tok)
        st.drafts[:, 0] = d
        for j in range(1, S):
            sb = DecodeBatch(tokens=st.tokens, lengths=(st.lengths + (j - 1)).contiguous(), req_pages=st.req_pages,
                             out_tokens=st.tokens)
            d, h_prev = self.mtp_step(sb, h_prev, d)
            h_prev = h_prev.contiguous()
            st.drafts[:, j] = d
        return st.out, st.accepted

    # ------------------------------------------------------------------- step --
    def decode_step(self, batch: DecodeBatch):
        """One decode step for every request of ``batch``: consumes ``batch.tokens``, writes
        the new KV / index entries, leaves greedy samples in ``batch.out_tokens`` and
        advances ``batch.lengths``."""
        import torch
        from ..ops import glue

        c = self.cfg
        self._mark("embed+begin")
        x = self.embed[batch.tokens.long()].contiguous()       # residual stream, updated in place
        new_ids = self.new_token_ids(batch)
        self._ctx = batch.lengths + 1                           # the new token attends to itself
        self.cache.begin_model_forward()
        delta = (None, 1, 0)             # (tensor, partial slots, slot stride): what the next norm adds to x
        for layer in range(c.layers):
            delta = self._layer(layer, self.layer_weights(layer), x, delta, batch, new_ids)
        self.cache.finish_model_forward()
        self._mark("lm_head+sample")
        idx = self._head(x, delta, batch.tokens.shape[0])
        self.last_hidden = x                                    # residual stream after the last layer (pre-norm)
        batch.out_tokens.copy_(idx)
        batch.lengths.add_(1)
        self._mark("end")
        return batch.out_tokens
