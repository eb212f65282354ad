"""GPU numerics for the first kernels: tcgen05 GEMM, radix top-k, record writers.
Each is compared with a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

from ulacache_b200.ops import _native as N
from ulacache_b200.ops import gemm, records, topk
from ulacache_b200.storage import layout as L

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,Nout,K,splits", [(16, 256, 128, 1), (64, 512, 1024, 1), (33, 384, 512, 2),
                                              (128, 1024, 2048, 4), (200, 7168, 2048, 0)])
def test_gemm_matches_reference(native, T, Nout, K, splits):
    torch.manual_seed(0)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(Nout, K, device="cuda", dtype=torch.bfloat16)
    status = N.new_status("cuda")
    y = gemm.linear(x, w, splits=splits, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "gemm")
    ref = gemm.linear_reference(x, w)
    err = (y.float() - ref).abs().max().item()
    assert err <= 0.02 * ref.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("T,heads", [(5, 3), (32, 16), (48, 128), (130, 4)])
def test_batched_gemm_with_quantising_epilogue(native, T, heads):
    """Per-head product whose epilogue quantises each head's 128 outputs as one fp8 group."""
    from ulacache_b200.ops import fp8

    torch.manual_seed(T + heads)
    x = torch.randn(T, heads, 512, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(heads, 128, 512, device="cuda") * 0.05).to(torch.bfloat16)
    status = N.new_status("cuda")
    q, sc = gemm.batched_linear_quant(x, w, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "gemm")
    ref = torch.einsum("tbk,bnk->tbn", x.float(), w.float()).reshape(T, heads * 128)
    want_q, want_s = fp8.act_quant_reference(ref)
    assert torch.allclose(sc, want_s, rtol=2e-3, atol=1e-6)
    got = q.view(torch.float8_e4m3fn).float().view(T, heads, 128) * sc.view(T, heads, 1)
    want = want_q.view(torch.float8_e4m3fn).float().view(T, heads, 128) * want_s.view(T, heads, 1)
    # one fp8 step (2^-3 relative) at most where the fp32 sums differ in the last bits
    assert (got - want).abs().max().item() <= 0.13 * want.abs().max().item()
    assert ((got - want).abs() > 1e-3 * want.abs().max()).float().mean().item() < 0.02


def test_per_head_products_at_prefill_row_counts(native, monkeypatch):
    """From 512 rows the per-head products take the library's batched GEMM; same results as the decode kernel
    (bf16 rounding of fp32 sums), head-interleaved inputs and both output layouts."""
    from ulacache_b200.ops import fp8

    torch.manual_seed(2)
    T, heads = 640, 8
    qb = torch.randn(T, heads * 192, device="cuda", dtype=torch.bfloat16)
    x = torch.as_strided(qb, (T, heads, 128), (qb.stride(0), 192, 1))             # the q_nope view of a fused projection
    w = (torch.randn(heads, 512, 128, device="cuda") * 0.05).to(torch.bfloat16)
    ref = torch.einsum("tbk,bnk->tbn", x.float(), w.float())
    out_a = torch.empty(T, heads, 512, device="cuda", dtype=torch.bfloat16)        # token-major: copied out of the product
    out_b = torch.empty(heads, T, 512, device="cuda", dtype=torch.bfloat16).transpose(0, 1)   # head-major storage: in place
    assert gemm.many_rows(T)
    gemm.batched_linear(x, w, out_a)
    gemm.batched_linear(x, w, out_b)
    monkeypatch.setenv("ULC_PREFILL_GEMM", "0")
    out_k = gemm.batched_linear(x, w, torch.empty(T, heads, 512, device="cuda", dtype=torch.bfloat16))
    monkeypatch.delenv("ULC_PREFILL_GEMM")
    torch.cuda.synchronize()
    tol = 0.02 * ref.abs().max().item()
    for got in (out_a, out_b, out_k):
        assert (got.float() - ref).abs().max().item() <= tol
    o_lat = torch.randn(T, heads, 512, device="cuda", dtype=torch.bfloat16)
    wv = (torch.randn(heads, 128, 512, device="cuda") * 0.05).to(torch.bfloat16)
    q, sc = gemm.batched_linear_quant(o_lat, wv)
    want_q, want_s = fp8.act_quant_reference(torch.einsum("tbk,bnk->tbn", o_lat.float(), wv.float()).reshape(T, heads * 128))
    assert torch.allclose(sc, want_s, rtol=2e-2, atol=1e-6)
    got = q.view(torch.float8_e4m3fn).float().view(T, heads, 128) * sc.view(T, heads, 1)
    want = want_q.view(torch.float8_e4m3fn).float().view(T, heads, 128) * want_s.view(T, heads, 1)
    assert (got - want).abs().max().item() <= 0.13 * want.abs().max().item()


@pytest.mark.parametrize("mode", ["row", "cluster", "rows", "rows_staged"])
@pytest.mark.parametrize("rows,Lmax,k", [(3, 100, 128), (4, 5000, 256), (2, 131072, 2048), (5, 40000, 2048),
                                         (32, 32768, 2048)])
def test_topk_matches_reference(native, rows, Lmax, k, mode):
    torch.manual_seed(1)
    s = torch.randn(rows, Lmax, device="cuda")
    lengths = torch.randint(max(1, Lmax // 2), Lmax + 1, (rows,), device="cuda", dtype=torch.int32)
    topk.set_launch_mode(mode)
    try:
        out = topk.topk(s, k, lengths)
        torch.cuda.synchronize()
    finally:
        topk.set_launch_mode("auto")
    ref = topk.topk_reference(s, k, lengths)
    for r in range(rows):
        assert sorted(out[r].tolist()) == sorted(ref[r].tolist())


@pytest.mark.parametrize("mode", ["row", "cluster", "rows", "rows_staged"])
def test_topk_narrow_score_range(native, mode):
    """Scores packed into one or two coarse bins (what ReLU-weighted index scores look like): the
    threshold bin then holds more elements than the shared-memory candidate store."""
    torch.manual_seed(5)
    s = 1.0 + 0.2 * torch.rand(3, 50000, device="cuda")
    s[2] = 1.5                      # every element tied: lowest positions win
    topk.set_launch_mode(mode)
    try:
        out = topk.topk(s, 2048)
        torch.cuda.synchronize()
    finally:
        topk.set_launch_mode("auto")
    ref = topk.topk_reference(s, 2048)
    for r in range(3):
        assert sorted(out[r].tolist()) == sorted(ref[r].tolist())


@pytest.mark.parametrize("mode", ["row", "cluster", "rows", "rows_staged"])
def test_topk_ties_and_transform(native, mode):
    s = torch.zeros(2, 9000, device="cuda")
    s[0, 100:200] = 1.0
    s[1, :] = 3.0
    table = (torch.arange(9000, device="cuda", dtype=torch.int32) * 2 + 7).repeat(2, 1)
    topk.set_launch_mode(mode)
    try:
        out = topk.topk(s, 512, xform=table)
        torch.cuda.synchronize()
    finally:
        topk.set_launch_mode("auto")
    ref = topk.topk_reference(s, 512, xform=table)
    for r in range(2):
        assert sorted(out[r].tolist()) == sorted(ref[r].tolist())


@pytest.mark.parametrize("rows,Lmax,k", [(3, 100, 128), (4, 5000, 256), (2, 131072, 2048), (5, 40000, 2048),
                                         (32, 32768, 2048), (130, 9000, 2048)])
def test_topk_histogram_method_matches_reference(native, rows, Lmax, k):
    """Histogram launch + selection launch through the global workspace (no clusters), twice in a row
    on the same workspace."""
    torch.manual_seed(3)
    for trial in range(2):
        s = torch.randn(rows, Lmax, device="cuda") if trial == 0 else 1.0 + 0.2 * torch.rand(rows, Lmax, device="cuda")
        if trial == 1:
            s[-1] = 1.5                                  # every element tied: lowest positions win
        lengths = torch.randint(max(1, Lmax // 2), Lmax + 1, (rows,), device="cuda", dtype=torch.int32)
        vals = torch.empty(rows, k, device="cuda")
        out = topk.topk(s, k, lengths, out_val=vals, method="hist")
        torch.cuda.synchronize()
        ref = topk.topk_reference(s, k, lengths)
        for r in range(rows):
            assert sorted(out[r].tolist()) == sorted(ref[r].tolist()), (trial, r)
            picked = out[r][out[r] >= 0].long()
            assert torch.equal(vals[r][out[r] >= 0], s[r][picked])
        assert topk.workspace_is_clean(topk.workspace(rows, "cuda"), rows)


def test_topk_many_rows_kernel(native):
    """The throughput kernel on what prefill and large batches give it: hundreds of rows (more rows than
    CTAs), ragged lengths around every internal boundary (k, the candidate store, chunk ends), rows whose
    stride breaks 16-byte alignment, heavy ties, -inf runs, values, candidate lists and the paged transform."""
    torch.manual_seed(11)
    rows, L, k = 330, 20011, 2048
    s = torch.randn(rows, L, device="cuda")
    s[5] = 0.25                                            # every element tied
    s[6, ::3] = 7.0                                        # a third of the row tied at the top
    s[7, 4000:] = float("-inf")
    s[8] = torch.rand(L, device="cuda").round(decimals=2)  # 101 distinct values
    lengths = torch.randint(1, L + 1, (rows,), device="cuda", dtype=torch.int32)
    for r, n in enumerate([0, 1, 2047, 2048, 2049, 8191, 8192, 8193, 16384, 16385, L]):
        lengths[10 + r] = n
    lengths[5:9] = L
    vals = torch.empty(rows, k, device="cuda")
    counts = torch.empty(rows, dtype=torch.int32, device="cuda")
    out = topk.topk(s, k, lengths, out_val=vals, out_count=counts)      # auto: this many rows take the throughput kernel
    torch.cuda.synchronize()
    ref = topk.topk_reference(s, k, lengths)
    for r in range(rows):
        assert sorted(out[r].tolist()) == sorted(ref[r].tolist()), r
        keep = out[r] >= 0
        assert torch.equal(vals[r][keep], s[r][out[r][keep].long()])
    assert torch.equal(counts.cpu(), lengths.clamp(max=k).cpu())
    for mode in ("rows", "rows_staged"):
        topk.set_launch_mode(mode)
        try:
            got = topk.topk(s, k, lengths)                          # the same rows through each form explicitly
            aligned = topk.topk(s[:, :20000].contiguous(), k)      # every row 16-byte aligned: all rows staged
            torch.cuda.synchronize()
        finally:
            topk.set_launch_mode("auto")
        assert all(sorted(got[r].tolist()) == sorted(ref[r].tolist()) for r in range(rows)), mode
        ref_a = topk.topk_reference(s[:40, :20000], k)
        assert all(sorted(aligned[r].tolist()) == sorted(ref_a[r].tolist()) for r in range(40)), mode
    topk.set_launch_mode("rows")
    try:
        # candidate-list mode with an index transform, few rows, explicit mode
        cv = torch.randn(3, 9000, device="cuda")
        ci = torch.randint(0, 50000, (3, 9000), device="cuda", dtype=torch.int32)
        got = topk.topk(cv, 512, in_idx=ci)
        want = topk.topk_reference(cv, 512, in_idx=ci)
        assert all(sorted(got[r].tolist()) == sorted(want[r].tolist()) for r in range(3))
        # long rows: several chunks, filter from samples
        big = torch.randn(4, 150001, device="cuda")
        got = topk.topk(big, 2048)
        want = topk.topk_reference(big, 2048)
        assert all(sorted(got[r].tolist()) == sorted(want[r].tolist()) for r in range(4))
        # a narrow range: the sample's filter bin holds most of the row (falls back to the exact pass over the row)
        narrow = 1.0 + 0.01 * torch.rand(3, 40000, device="cuda")
        got = topk.topk(narrow, 2048)
        want = topk.topk_reference(narrow, 2048)
        assert all(sorted(got[r].tolist()) == sorted(want[r].tolist()) for r in range(3))
    finally:
        topk.set_launch_mode("auto")


def _single_rank_view(pool, directory, rec_bytes):
    return records.make_pool_view(hbm_ptrs=[pool.data_ptr()], dir_ptrs=[directory.data_ptr()], host_ptr=0,
                                  dir_len=directory.numel(), hbm_slots=pool.shape[0], host_slots=0,
                                  rec_bytes=rec_bytes, owners=L.OwnerMap(1, 6), my_rank=0)


@pytest.mark.parametrize("fmt", ["mla.scaled656.fp8.v1", "mla.raw576.fp8.v1", "mla.bf16.1152.v1"])
def test_kv_write_matches_reference(native, fmt):
    torch.manual_seed(2)
    plane = L.record_plane(fmt)
    T, slots = 300, 512
    pool = torch.zeros(slots, plane.bytes_per_record, dtype=torch.uint8, device="cuda")
    directory = torch.full((1024,), -1, dtype=torch.int32, device="cuda")
    ids = torch.randperm(900, device="cuda")[:T].to(torch.int32) + 1
    slot_of = torch.randperm(slots, device="cuda")[:T].to(torch.int32)
    directory[ids.long()] = slot_of
    latent = torch.randn(T, 512, device="cuda", dtype=torch.bfloat16) * 3
    rope = torch.randn(T, 64, device="cuda", dtype=torch.bfloat16)
    status = N.new_status("cuda")
    records.kv_write(_single_rank_view(pool, directory, plane.bytes_per_record),
                     L.KERNEL_FORMAT_CODE[fmt], latent, rope, ids, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "kv_write")
    got = records.DECODERS[fmt](pool[slot_of.long()])
    truth = torch.cat([latent, rope], dim=1).float()
    # e4m3 keeps 3 mantissa bits: half a step is 1/16 of the value; bf16 formats are exact
    err = (got - truth).abs()
    bound = truth.abs() / 16 + 0.03 if "fp8" in fmt else torch.zeros_like(truth)
    if fmt == "mla.scaled656.fp8.v1":
        bound[:, 512:] = 0
    assert (err <= bound).all(), (err - bound).max().item()
    exact = (pool[slot_of.long()] == records.ENCODERS[fmt](latent, rope)).float().mean().item()
    assert exact > 0.99, exact


@pytest.mark.parametrize("fused", [False, True])
def test_index_key_store(native, fused):
    torch.manual_seed(3)
    T, pages = 500, 16
    pool = torch.zeros(pages, L.INDEX_PAGE_BYTES, dtype=torch.uint8, device="cuda")
    ids = torch.randperm(pages * 64 - 1, device="cuda")[:T].to(torch.int32) + 1
    k = torch.randn(T, 128, device="cuda", dtype=torch.bfloat16)
    kw = {}
    if fused:
        kw = dict(gamma=torch.rand(128, device="cuda") + 0.5, beta=torch.randn(128, device="cuda") * 0.1,
                  cos_sin=torch.cat([torch.cos(torch.rand(64, 32, device="cuda")), torch.sin(torch.rand(64, 32, device="cuda"))], 1).contiguous(),
                  positions=torch.randint(0, 64, (T,), device="cuda", dtype=torch.int32))
    iv = records.make_index_view(page_ptrs=[pool.data_ptr()], pages_per_rank=pages, ranks=1, my_rank=0)
    status = N.new_status("cuda")
    records.index_key_store(iv, k, ids, status=status, **kw)
    torch.cuda.synchronize()
    N.raise_on_status(status, "index_key_store")
    keys, scales = records.decode_index_page(pool)
    q, sc = records.encode_index_key(k, **kw)
    want = q.view(torch.float8_e4m3fn).float() * sc[:, None]
    got = keys.view(-1, 128)[ids.long()] * scales.view(-1)[ids.long()][:, None]
    assert torch.allclose(got, want, rtol=0.08, atol=2e-2)
