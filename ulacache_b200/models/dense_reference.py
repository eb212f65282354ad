"""A plain PyTorch statement of the DSA MoE decode step, written independently of the kernels.

The oracle for the composed model: it keeps every request's KV and index history as dense
tensors, uses dequantised weights, and computes attention the textbook way - per head keys and
values are materialised from the latent (``k_nope = latent @ W_UK``, ``v = latent @ W_UV``) instead
of absorbing ``W_UK`` into the query and ``W_UV`` into the output as the kernels do, and the softmax
runs over the selected tokens of a dense score matrix.  Quantisation points (fp8 activations,
fp8 KV records, fp8 index keys and queries, bf16 tensors between stages) are the model's, applied
with ``torch`` casts, so the two agree to accumulation-order noise.

Single rank only (``tp == 1``); used by ``tests/test_gpu_model_oracle.py``.

The reference library has no model; this file has no counterpart there.
"""
from __future__ import annotations

from typing import List, Optional


def _bf16(x):
    import torch

    return x.to(torch.bfloat16).float()


def _fake_quant_act(x):
    """Per (row, 128 columns) fp8 e4m3 quantise / dequantise of a bf16-rounded activation."""
    import torch

    m, k = x.shape
    g = _bf16(x).view(m, k // 128, 128)
    amax = g.abs().amax(dim=-1, keepdim=True)
    scale = torch.div(torch.clamp(amax, min=1e-4), torch.full_like(amax, 448.0))
    q = (g * (1.0 / scale)).to(torch.float8_e4m3fn).float()
    return (q * scale).view(m, k)


def _rms(x, w, eps):
    import torch

    xf = x.float()
    return _bf16(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float())


def _rope_pairs(x, cos, sin):
    """Rotate pairs (i, i + d/2) of the last dimension (d = x.shape[-1]); bf16 result."""
    import torch

    d = x.shape[-1] // 2
    a, b = x[..., :d], x[..., d:]
    return _bf16(torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1))


def _dequant_linear(lin):
    """Canonical fp32 [nout, k] weight of a block-scaled fp8 linear."""
    from ..ops import fp8

    w = fp8.dequantize_weight(fp8.untile_weight(lin.q), lin.s)
    return w[: lin.nout].float()


class DenseReferenceDecoder:
    def __init__(self, model):
        import torch
        from ..ops import fp8

        if model.tp != 1:
            raise ValueError("the dense reference covers one rank")
        self.cfg = c = model.cfg
        self.model = model
        self.device = model.device
        self.layers = []
        for l in range(c.layers):
            w = model.layer_weights(l)
            d = dict(dense=w.dense, attn_norm=w.attn_norm.float(), ffn_norm=w.ffn_norm.float(),
                     q_norm=w.q_norm.float(), kv_norm=w.kv_norm.float(), w_in=_dequant_linear(w.w_in),
                     w_qb=_dequant_linear(w.w_qb), w_o=_dequant_linear(w.w_o),
                     w_uk=w.w_uk_t.float(),            # [heads, 512, 128]: k_nope[h] = latent @ w_uk[h]
                     w_uv=w.w_uv_t.float(),            # [heads, 128, 512]: v[h] = w_uv[h] @ latent
                     gamma=w.index_gamma.float(), beta=w.index_beta.float())
            if w.dense:
                d["w13"], d["w2"] = _dequant_linear(w.w13), _dequant_linear(w.w2)
            else:
                d["router"] = w.router.float()
                d["router_bias"] = w.router_bias.float()
                d["e13"] = fp8.dequantize_weight(fp8.untile_weight(w.e13_q), w.e13_s).float()     # [E(+1), 2F, H]
                d["e2"] = fp8.dequantize_weight(fp8.untile_weight(w.e2_q), w.e2_s).float()        # [E(+1), H, F]
                d["shared_fused"] = w.shared_fused
                d["n_routed"] = w.local_experts
            self.layers.append(d)
        self.embed = model.embed.float()
        self.final_norm = model.final_norm.float()
        self.lm_head = _dequant_linear(model.lm_head)
        self.cos, self.sin = model.cos.float(), model.sin.float()
        # history[layer][request] = dict(latent [T,512], rope [T,64], ikey [T,128]) as the records decode
        self.history: List[List[dict]] = []
        self.selections = None

    # ------------------------------------------------------------------ history --
    def start(self, n_requests: int):
        import torch

        z = lambda d: torch.zeros((0, d), dtype=torch.float32, device=self.device)
        self.history = [[dict(latent=z(512), rope=z(64), ikey=z(128)) for _ in range(n_requests)]
                        for _ in range(self.cfg.layers)]

    @staticmethod
    def _stored_kv(latent, rope):
        """What a scaled656 record gives back for (latent, rope)."""
        from ..ops import records

        dec = records.decode_scaled656(records.encode_scaled656(latent, rope))
        return dec[:, :512], dec[:, 512:]

    @staticmethod
    def _stored_index_key(k, **kw):
        import torch
        from ..ops import records

        q, scale = records.encode_index_key(k, **kw)
        return q.view(torch.float8_e4m3fn).float() * scale.unsqueeze(-1)

    def append_history(self, layer: int, request: int, latent, rope, index_key, *, raw_index_key=True):
        """Append tokens written straight into the cache (a synthetic prefill): ``latent`` / ``rope`` as
        given to ``cache.write``, ``index_key`` as given to ``index_key_store`` (no norm, no rotary)."""
        import torch

        h = self.history[layer][request]
        lat, rp = self._stored_kv(latent, rope)
        ik = self._stored_index_key(index_key) if raw_index_key else index_key
        h["latent"] = torch.cat([h["latent"], lat])
        h["rope"] = torch.cat([h["rope"], rp])
        h["ikey"] = torch.cat([h["ikey"], ik])

    # --------------------------------------------------------------------- step --
    def _attention(self, l: int, d: dict, hq, positions, selections):
        import torch

        c = self.cfg
        B = hq.shape[0]
        fused = _bf16(hq @ d["w_in"].t())
        o0, o1, o2, o3 = c.q_lora, c.q_lora + c.kv_lora, c.q_lora + c.kv_lora + c.rope_dim, \
            c.q_lora + c.kv_lora + c.rope_dim + c.index_dim
        q_a, kv_a, k_pe, ik_raw, iw_raw = fused[:, :o0], fused[:, o0:o1], fused[:, o1:o2], fused[:, o2:o3], \
            fused[:, o3:o3 + c.index_heads]
        cos, sin = self.cos[positions.long()], self.sin[positions.long()]               # [B, 32]
        qn = _fake_quant_act(_rms(q_a, d["q_norm"], c.rms_eps))
        qb = _bf16(qn @ d["w_qb"].t())
        q = qb[:, : c.heads * 192].view(B, c.heads, 192)
        q_nope, q_pe = q[..., :128], _rope_pairs(q[..., 128:], cos.unsqueeze(1), sin.unsqueeze(1))
        iq = qb[:, c.heads * 192:].view(B, c.index_heads, c.index_dim).clone()
        iq[..., :64] = _rope_pairs(iq[..., :64], cos.unsqueeze(1), sin.unsqueeze(1))
        # indexer queries are fp8 per head; the head weight carries the scale and 1 / sqrt(heads)
        amax = iq.abs().amax(dim=-1, keepdim=True)
        iscale = torch.div(torch.clamp(amax, min=1e-4), torch.full_like(amax, 448.0))
        iq_q = (iq * (1.0 / iscale)).to(torch.float8_e4m3fn).float()
        iw = iw_raw * (c.index_heads ** -0.5) * iscale.squeeze(-1)                       # [B, 64]
        # this token's KV record and index key, as stored
        latent = _rms(kv_a, d["kv_norm"], c.rms_eps)
        k_rope = _rope_pairs(k_pe, cos, sin)
        lat_s, rope_s = self._stored_kv(latent, k_rope)
        from ..ops import records

        cos_sin = torch.cat([self.cos, self.sin], dim=1)
        q8, sc = records.encode_index_key(ik_raw, gamma=d["gamma"], beta=d["beta"], cos_sin=cos_sin, positions=positions)
        ikey_s = q8.view(torch.float8_e4m3fn).float() * sc.unsqueeze(-1)
        out = torch.zeros((B, c.heads * c.v_dim), dtype=torch.float32, device=hq.device)
        chosen = []
        for b in range(B):
            h = self.history[l][b]
            h["latent"] = torch.cat([h["latent"], lat_s[b:b + 1]])
            h["rope"] = torch.cat([h["rope"], rope_s[b:b + 1]])
            h["ikey"] = torch.cat([h["ikey"], ikey_s[b:b + 1]])
            T = h["latent"].shape[0]
            # index scores over the whole context (the key's fp8 scale is already inside ikey)
            s = torch.relu(torch.einsum("hd,td->ht", iq_q[b], h["ikey"]))
            logit = (s * iw[b].unsqueeze(-1)).sum(dim=0)                                    # [T]
            if selections is not None:
                sel = selections[l][b]
                sel = sel[sel >= 0].long()
            elif T <= c.topk:
                sel = torch.arange(T, device=hq.device)
            else:
                sel = torch.topk(logit, c.topk).indices
            chosen.append((logit, sel))
            lat_sel, rope_sel = h["latent"][sel], h["rope"][sel]                           # [S,512], [S,64]
            k_nope = torch.einsum("sc,hcd->hsd", lat_sel, d["w_uk"])                      # [heads, S, 128]
            v = torch.einsum("sc,hdc->hsd", lat_sel, d["w_uv"])                           # [heads, S, 128]
            scores = torch.einsum("hd,hsd->hs", q_nope[b], k_nope) + torch.einsum("hd,sd->hs", q_pe[b], rope_sel)
            p = torch.softmax(scores * c.softmax_scale, dim=-1)
            out[b] = torch.einsum("hs,hsd->hd", p, v).reshape(-1)
        self._last_index = chosen
        oq = _fake_quant_act(out)
        return _bf16(oq @ d["w_o"].t())

    def _ffn(self, d: dict, h, hq, pinned_choice=None):
        import torch

        c = self.cfg
        if d["dense"]:
            mid = _bf16(hq @ d["w13"].t())
            f = mid.shape[1] // 2
            act = _fake_quant_act(torch.nn.functional.silu(mid[:, :f]) * mid[:, f:])
            return _bf16(act @ d["w2"].t())
        logits = _bf16(h @ d["router"].t())
        sc = torch.sigmoid(logits)
        choice = torch.topk(sc + d["router_bias"], c.experts_per_token, dim=-1).indices
        self.routing.append((sc, choice))
        if pinned_choice is not None:           # random-init routers score all experts nearly alike: near-ties
            choice = pinned_choice.long()       # are the rule, so the experts can be pinned to the kernels' choice
        g = torch.gather(sc, 1, choice)
        g = g / g.sum(-1, keepdim=True) * c.routed_scale
        out = torch.zeros_like(h)

        def expert(e, rows):
            mid = _bf16(rows @ d["e13"][e].t())
            f = mid.shape[1] // 2
            act = _fake_quant_act(torch.nn.functional.silu(mid[:, :f]) * mid[:, f:])
            return _bf16(act @ d["e2"][e].t())

        for b in range(h.shape[0]):
            acc = torch.zeros(c.hidden, dtype=torch.float32, device=h.device)
            if d["shared_fused"]:
                acc = acc + expert(d["n_routed"], hq[b:b + 1])[0]
            for j in range(c.experts_per_token):
                acc = acc + g[b, j] * expert(int(choice[b, j]), hq[b:b + 1])[0]
            out[b] = acc
        return _bf16(out)

    def step(self, tokens, positions, selections=None, routing=None):
        """One decode step: ``tokens`` [B] at ``positions`` [B] (tokens already in each request's
        cache).  ``selections[layer][b]``: optional record positions to attend to (to pin the oracle
        to the very selection the kernels made); by default the oracle takes its own top-k.
        Returns fp32 logits [B, vocab] and appends the step's KV / index entries to the history."""
        import torch

        c = self.cfg
        x = self.embed[tokens.long()].clone()                  # bf16-valued residual stream
        delta = None
        self.sublayers = []                                    # (attention output, feed-forward output) per layer
        self.routing = []                                      # (expert scores, own choice) per MoE layer
        moe_seen = 0
        for l, d in enumerate(self.layers):
            if delta is not None:
                x = _bf16(x + delta)
            h = _rms(x, d["attn_norm"], c.rms_eps)
            attn = self._attention(l, d, _fake_quant_act(h), positions, selections)
            x = _bf16(x + attn)
            h2 = _rms(x, d["ffn_norm"], c.rms_eps)
            pin = None
            if routing is not None and not d["dense"]:
                pin = routing[moe_seen][0]
                moe_seen += 1
            delta = self._ffn(d, h2, _fake_quant_act(h2), pin)
            self.sublayers.append((attn, delta))
        x = _bf16(x + delta)
        hf = _fake_quant_act(_rms(x, self.final_norm, c.rms_eps))
        return _bf16(hf @ self.lm_head.t())[:, : c.vocab]
