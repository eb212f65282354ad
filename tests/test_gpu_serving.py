"""End-to-end serving loop on the GPU with the tiny model: prefill through the decode kernels, prefix
reuse through the radix tree, a device tier smaller than the working set (host tier exercised)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_prefill_matches_token_by_token_decode_and_prefix_is_reused(native, monkeypatch):
    monkeypatch.setenv("ULC_DETERMINISTIC", "1")        # sorted selections: bit-reproducible attention
    from ulacache_b200.models.dsa_moe import DsaMoeConfig
    from ulacache_b200.serving.server import ServingEngine

    cfg = DsaMoeConfig().tiny(layers=2, topk=128)
    torch.manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (200,)).tolist()

    def run(chunk):
        srv = ServingEngine(cfg, max_batch=4, max_context=512, device_records=4096, host_records=8192, prefill_chunk=chunk)
        t = [0.0]
        srv.clock = lambda: t[0]
        srv.submit(1, prompt, 6, 0.0)
        while srv.busy():
            srv.step()
            t[0] += 1.0
        toks = list(srv.finished[0].generated)
        return srv, toks

    # (both chunk sizes use the GEMM's 16-row geometry: other geometries sum K blocks in another
    # order and agree only to fp32 rounding)
    srv_a, a = run(8)           # prompt in chunks of 8 rows
    srv_b, b = run(1)           # prompt one token at a time (plain decode)
    assert a == b and len(a) == 6
    srv_b.close()
    # a second request with the same first 128 tokens starts from the cached pages
    srv_a.submit(2, prompt[:150] + [5, 6, 7], 3, 100.0)
    t = [100.0]
    srv_a.clock = lambda: t[0]
    while srv_a.busy():
        srv_a.step()
    rep = srv_a.report()
    assert rep["finished_requests"] == 2 and rep["reused_prefix_tokens"] == 128 and rep["unserved"] == 0
    assert rep["prefill_tokens"] == 200 + (153 - 128)
    srv_a.close()


def test_snapshot_bank_restores_a_cache_that_decodes_the_same_tokens(native, tmp_path):
    """fill -> save (two owner shards, KV + index planes) -> restore into a fresh engine -> both decode the
    same tokens over eight steps."""
    from ulacache_b200.experiments import kv_bank

    assert kv_bank.main(["--tiny", "--layers", "3", "--batch", "3", "--prompt-len", "700", "--steps", "8",
                         "--dir", str(tmp_path / "bank")]) == 0


def test_recorded_trajectory_replays_through_the_decode_engine(native, monkeypatch):
    """Record six natural greedy steps, then replay them into a fresh engine: the engine presents the same
    requests at the same positions every step, decodes the recorded tokens, and produces the same samples."""
    monkeypatch.setenv("ULC_DETERMINISTIC", "1")
    from ulacache_b200.models.dsa_moe import DsaMoeConfig
    from ulacache_b200.serving.engine import DecodeEngine
    from ulacache_b200.tools.fixed_output import ReplayMismatch, ReplayTrace, TraceTokenReplay

    cfg = DsaMoeConfig().tiny(layers=2)
    B, prompt, steps = 3, 200, 6

    def engine():
        e = DecodeEngine(cfg, batch=B, prompt_len=prompt, max_new_tokens=steps + 2, use_graph=False)
        e.fill_synthetic()
        return e

    eng = engine()
    first = eng.batch.tokens.clone()
    natural = []
    for _ in range(steps):
        out = eng.step_device()
        natural.append(out.clone())
        eng.batch.tokens.copy_(out)
    eng.close()
    keys = [f"r0.{i}" for i in range(B)]
    outputs = {k: [int(natural[s][i]) for s in range(steps)] for i, k in enumerate(keys)}
    trace = ReplayTrace.from_token_run(attention_dp=1, repeat=0, rank=0, keys=keys, input_tokens=[prompt] * B,
                                       outputs=outputs)

    eng2 = engine()
    eng2.batch.tokens.copy_(first)
    rp = TraceTokenReplay(trace, attention_dp=1, rank=0)
    seen = []
    orig = rp.sample
    rp.sample = lambda nat: (seen.append(nat.clone()), orig(nat))[1]
    receipt = eng2.run_replay(rp, "cohort", keys=keys)
    assert receipt["complete"] and receipt["frames"] == steps and receipt["forward_calls"] == steps
    assert all(torch.equal(a, b) for a, b in zip(seen, natural))       # same inputs, same model: same samples
    with pytest.raises((ReplayMismatch, RuntimeError)):                 # the recording is used up
        eng2.run_replay(rp, "cohort", keys=keys, steps=1)
    eng2.close()
