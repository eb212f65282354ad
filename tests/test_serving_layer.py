import pytest
import torch

from ulacache_b200.serving.admission import AdmissionController, CacheBudget
from ulacache_b200.serving.allocator import LogicalPageAllocator, OutOfLogicalPages
from ulacache_b200.serving.hooks import SharedIndexAdapter
from ulacache_b200.serving.radix_tree import RadixPrefixTree


def test_radix_match_insert_evict():
    t = RadixPrefixTree(page_tokens=4)
    a = list(range(12))
    assert t.insert(a, [10, 11, 12]) == []
    b = a[:8] + [99, 98, 97, 96, 5]
    m = t.match(b)
    assert [n.page for n in m] == [10, 11]
    assert t.insert(b, [10, 11, 20]) == [] and t.cached_pages() == 4
    assert t.insert(a, [10, 11, 77]) == [77]                 # duplicate of a cached page is handed back
    t.lock(m)
    t.match(a)                                                # page 12 is now more recent than page 20
    assert t.evict(1) == [20]
    assert t.evict(5) == [12]                                 # 10 and 11 are locked
    t.unlock(m)
    assert sorted(t.evict(5)) == [10, 11] and t.cached_pages() == 0


class _Tier:
    def __init__(self):
        self.live = set()

    def register(self, ids):
        assert not (set(ids.tolist()) & self.live)
        self.live |= set(ids.tolist())

    def release(self, ids):
        assert set(ids.tolist()) <= self.live
        self.live -= set(ids.tolist())


def test_allocator_evicts_cached_prefixes_when_short():
    tier = _Tier()
    alloc = LogicalPageAllocator(owners=2, device_pages=2, host_pages=1, tier=tier)
    assert alloc.token_capacity == 5 * 64 and alloc.available_pages() == 5
    p = alloc.alloc(3)
    assert 0 not in p and len(tier.live) == 3 * 64
    alloc.tree.insert(list(range(128)), p[:2])                # request finished: two pages stay as a cached prefix
    alloc.free_pages(p[2:])
    q = alloc.alloc(4)                                        # 3 free + 1 evicted from the tree
    assert len(q) == 4 and alloc.tree.cached_pages() == 1 and len(tier.live) == 5 * 64
    with pytest.raises(OutOfLogicalPages):
        alloc.alloc(3)


def test_admission_budget():
    adm = AdmissionController(CacheBudget(owners=8, device_records=64 * 100, host_records=64 * 300,
                                          prefill_window_records=4096, max_running_requests=2))
    assert adm.budget.token_capacity == 8 * 64 * 400 - 64
    assert adm.admit(1, 100_000, 1024)
    assert not adm.can_admit(110_000, 1024)
    assert adm.can_admit(110_000, 1024, reusable_prefix=64 * 200)
    assert adm.admit(2, 1000, 24) and not adm.can_admit(10, 10)        # running cap
    adm.finish(1)
    assert adm.used_tokens == 1024 and adm.prefill_chunk_fits(4000, 96) and not adm.prefill_chunk_fits(4000, 97)
    assert adm.largest_prefill_chunk(4000, 8192) == 96


class _Client:
    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        return lambda *a, **k: self.calls.append((name, a[0] if a else None)) or "view"


def test_hook_surface_order_and_selection_reuse():
    c = _Client()
    ad = SharedIndexAdapter(c, 3, selection_owner=(0, 0, 2), topk=128, prefill_window_records=4096)
    ad.prepare_batch(current_ids="cur")
    ad.on_index_ready(0)
    ad.prepare_topk_lookup(0, "sel0")
    assert ad.prepare_packed_attention(0, "ids", "vals") == "view"
    ad.after_attention(0)
    ad.before_layer_prepare(1)
    ad.reuse_selection(1)
    ad.prepare_packed_attention(1)
    ad.after_attention(1)
    with pytest.raises(KeyError):
        ad.reuse_selection(2)
    ad.finish_batch()
    assert [n for n, _ in c.calls] == ["begin_model_forward", "prepare_sparse_attention", "write",
                                       "get_resident_attention_inputs", "finish_layer_attention",
                                       "prepare_sparse_attention", "get_resident_attention_inputs",
                                       "finish_layer_attention", "finish_model_forward"]
    chunks = ad.prepare_extend(10_000, cached_prefix=64, chunk_tokens=2048)
    assert sum(ch.tokens for ch in chunks) == 10_000 - 64 and all(ch.window_records <= 4096 for ch in chunks)


def test_entry_point_writes_the_startup_receipt(tmp_path):
    import json
    import os
    import subprocess
    import sys

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(repo, "ulacache_b200", "config", "models", "b200-native-dpa.json")
    for rank in (0, 1):
        env = dict(os.environ, RANK=str(rank))
        res = subprocess.run([sys.executable, "-m", "ulacache_b200.serving.entry", "--config", cfg, "--layers", "2",
                              "--device", "cpu", "--scale", "0.001", "--audit-dir", str(tmp_path)], cwd=repo, env=env,
                             capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stderr[-1500:]
    out = subprocess.run([sys.executable, "-m", "ulacache_b200.experiments.capacity", "--audit-dir", str(tmp_path)],
                         cwd=repo, capture_output=True, text=True, timeout=120)
    rep = json.loads(out.stdout.strip().splitlines()[-1])
    assert rep["ranks"] == 2 and rep["device_records"] == 2 * 1024 and rep["host_records"] == 2 * 3136
    assert rep["unique_kv_records"] == rep["device_records"] + rep["host_records"]


def test_launcher_resolves_methods_and_capacity(capsys):
    """The per-method launcher: layouts, tier sizes and the capacity each method admits under one budget."""
    from ulacache_b200.serving import launch

    ns = lambda **kw: __import__("argparse").Namespace(**dict(dict(
        method="ulacache", mode="dpa", batch_per_gpu=32, prompt_len=32768, max_new_tokens=64, layers=0, hot_buffer=4096,
        host_fraction=0.0, kv_budget_hbm_gb=64.0, kv_budget_host_gb=128.0), **kw))
    dpa = launch.resolve(ns(), 8)
    assert (dpa["mode"], dpa["kv_layout"], dpa["batch_per_engine"], dpa["global_batch"]) == ("dpa", "pooled", 32, 256)
    tp = launch.resolve(ns(mode="tp"), 8)
    assert tp["batch_per_engine"] == 256 and tp["records_per_rank"] < dpa["records_per_rank"] * 1.02
    hic = launch.resolve(ns(method="hicache"), 8)
    assert (hic["mode"], hic["kv_layout"]) == ("tp", "replicated") and hic["records_per_rank"] > 7.9 * tp["records_per_rank"]
    his = launch.resolve(ns(method="hisparse"), 8)
    assert his["device_record_capacity"] == 256 * 4096 and his["host_record_capacity"] > his["records_per_rank"] - 256 * 4096
    cap = {m: launch.capacity(ns(method=m), 8)["tokens_admitted"] for m in launch.METHODS}
    assert cap["ulacache"] == 8 * cap["hicache"] and cap["hisparse"] < cap["hicache"]
    assert launch.main(["--method", "hicache", "--dry-run"]) == 0
    assert '"kv_layout": "replicated"' in capsys.readouterr().out
