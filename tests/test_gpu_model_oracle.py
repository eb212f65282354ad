"""The composed decode step against an independent dense PyTorch decoder.

Every kernel has its own fp32 reference; this test pins the COMPOSITION (projection splits, rotary
conventions, the absorbed form of MLA attention, indexer scoring and selection, routing, expert
combine, residual wiring): logits of ``DsaMoeModel.decode_step`` must match
``DenseReferenceDecoder`` (dequantised weights, keys and values materialised per head, dense
attention over the selected tokens) step after step, and the greedy tokens must agree."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _positions_of(ids_by_request, sel, span):
    """Selected logical record IDs [B, k] -> positions inside each request (-1 stays -1)."""
    out = []
    for b, ids in enumerate(ids_by_request):
        lut = torch.full((int(ids.max()) + 1,), -1, dtype=torch.long, device=ids.device)
        lut[ids.long()] = torch.arange(ids.numel(), device=ids.device)
        row = sel[b].long()
        ok = (row >= 0) & (row < lut.numel())
        out.append(torch.where(ok, lut[row.clamp(min=0, max=lut.numel() - 1)], torch.full_like(row, -1)))
    return out


@pytest.mark.parametrize("prompt", [90, 300])          # below and above the top-k of the tiny model (128)
def test_decode_step_matches_dense_reference(native, monkeypatch, prompt):
    from ulacache_b200.models.dense_reference import DenseReferenceDecoder
    from ulacache_b200.models.dsa_moe import DsaMoeConfig
    from ulacache_b200.serving.engine import DecodeEngine

    monkeypatch.setenv("ULC_DETERMINISTIC", "1")
    cfg = DsaMoeConfig().tiny(layers=3)                 # one dense layer and two MoE layers
    B, steps = 3, 8
    eng = DecodeEngine(cfg, batch=B, prompt_len=prompt, max_new_tokens=steps + 4, use_graph=False)
    ref = DenseReferenceDecoder(eng.model)
    ref.start(B)

    def keep(layer, first, last, lat, rope, key):
        assert first == 0 and last == B * prompt
        for b in range(B):
            sl = slice(b * prompt, (b + 1) * prompt)
            ref.append_history(layer, b, lat[sl], rope[sl], key[sl])

    eng.fill_synthetic(on_chunk=keep)
    span = 64
    # logical IDs of every position a request can reach (prompt + generated)
    pages = eng.batch.req_pages.long()
    reach = prompt + steps + 1
    pos = torch.arange(reach, device=eng.device)
    ids_by_request = [(pages[b, pos // span] * span + pos % span) for b in range(B)]
    worst, mismatched = 0.0, 0
    for step in range(steps):
        tokens = eng.batch.tokens.clone()
        positions = eng.batch.lengths.clone()
        eng.model.record_selections, eng.model.record_routing = [], []
        eng.step_device()
        torch.cuda.synchronize()
        eng.check()
        got = eng.model.last_logits[:, : cfg.vocab].float()
        sels = [_positions_of(ids_by_request, s, span) for s in eng.model.record_selections]
        routing = eng.model.record_routing
        eng.model.record_selections = eng.model.record_routing = None
        assert len(sels) == cfg.layers and len(routing) == cfg.layers - cfg.dense_layers
        want = ref.step(tokens, positions, selections=sels, routing=routing)
        # (fp8 activations turn last-bit differences of accumulation order into whole quantisation steps,
        # so the composed logits agree to a few per cent; a wrong wiring shows as tens of per cent)
        # the kernels' experts are the oracle's own choice, up to near-ties of the (random-init) router
        for (choice, gate), (scores, own) in zip(routing, ref.routing):
            picked = torch.gather(scores, 1, choice.long())
            kth = torch.gather(scores, 1, own)[:, -1:]
            assert bool((picked >= kth - 2e-2).all())            # router logits are bf16
            g = picked / picked.sum(-1, keepdim=True) * cfg.routed_scale
            assert torch.allclose(gate, g, rtol=2e-2, atol=1e-3)
        err = (got - want).abs().max().item()
        scale = want.abs().max().item()
        worst = max(worst, err / scale)
        rms = ((got - want).norm() / want.norm()).item()
        # worst element within 12 % of the largest logit and the whole matrix within 10 % relative rms
        # (the noise measured across accumulation orders is 4 to 9 % and 4 to 7 %)
        assert err <= 0.12 * scale + 1e-3 and rms <= 0.10, (step, err, scale, rms)
        # greedy tokens agree unless the oracle's two best logits are within the tolerance
        top2 = torch.topk(want, 2, dim=-1).values
        gap = (top2[:, 0] - top2[:, 1])
        same = eng.batch.out_tokens.long() == want.argmax(dim=-1)
        assert bool((same | (gap <= 0.12 * scale)).all()), (step, eng.batch.out_tokens.tolist(), want.argmax(-1).tolist())
        mismatched += int((~same).sum())
    assert mismatched <= steps * B // 4, mismatched        # (a tiny random-init model has many near-tied logits)
    eng.close()


def test_selection_is_the_oracles_topk(native, monkeypatch):
    """The record IDs the indexer + radix select choose are the dense oracle's top-k of its own
    index scores (differences only among scores within rounding of the k-th)."""
    from ulacache_b200.models.dense_reference import DenseReferenceDecoder
    from ulacache_b200.models.dsa_moe import DsaMoeConfig
    from ulacache_b200.serving.engine import DecodeEngine

    monkeypatch.setenv("ULC_DETERMINISTIC", "1")
    cfg = DsaMoeConfig().tiny(layers=2)
    B, prompt = 2, 400
    eng = DecodeEngine(cfg, batch=B, prompt_len=prompt, max_new_tokens=8, use_graph=False)
    ref = DenseReferenceDecoder(eng.model)
    ref.start(B)

    def keep(layer, first, last, lat, rope, key):
        for b in range(B):
            sl = slice(b * prompt, (b + 1) * prompt)
            ref.append_history(layer, b, lat[sl], rope[sl], key[sl])

    eng.fill_synthetic(on_chunk=keep)
    pages = eng.batch.req_pages.long()
    pos = torch.arange(prompt + 4, device=eng.device)
    ids_by_request = [(pages[b, pos // 64] * 64 + pos % 64) for b in range(B)]
    tokens, positions = eng.batch.tokens.clone(), eng.batch.lengths.clone()
    eng.model.record_selections = []
    eng.step_device()
    torch.cuda.synchronize()
    sels = [_positions_of(ids_by_request, s, 64) for s in eng.model.record_selections]
    # layer 0 sees the same inputs in both implementations: compare there with the oracle's own choice
    ref.step(tokens, positions, selections=None)
    # (the oracle recorded (scores, own selection) of its LAST layer; rerun layer 0 alone for the check)
    ref2 = DenseReferenceDecoder(eng.model)
    ref2.history = [[dict(latent=h["latent"][:-1], rope=h["rope"][:-1], ikey=h["ikey"][:-1]) for h in layer]
                    for layer in ref.history]
    ref2.layers = ref2.layers[:1]
    ref2.cfg = cfg
    x = ref2.embed[tokens.long()]
    from ulacache_b200.models import dense_reference as D

    h = D._rms(x, ref2.layers[0]["attn_norm"], cfg.rms_eps)
    ref2._attention(0, ref2.layers[0], D._fake_quant_act(h), positions, None)
    for b in range(B):
        logit, own = ref2._last_index[b]
        mine = set(own.tolist())
        theirs = set(p for p in sels[0][b].tolist() if p >= 0)
        assert len(theirs) == cfg.topk
        diff = mine ^ theirs
        kth = torch.topk(logit, cfg.topk).values[-1].item()
        for p in diff:                                   # only near-ties at the cut may differ
            assert abs(logit[p].item() - kth) <= 2e-2 * max(1.0, abs(kth)), (b, p, logit[p].item(), kth)
        assert len(diff) <= 8, len(diff)
    eng.close()
