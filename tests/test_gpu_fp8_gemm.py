"""Block-scaled fp8 grouped GEMM and the activation quantiser against fp32 references."""
import pytest
import torch

from ulacache_b200.ops import _native as N
from ulacache_b200.ops import fp8

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("swiglu", [False, True])
def test_act_quant(native, swiglu):
    torch.manual_seed(0)
    x = torch.randn(37, 512 * (2 if swiglu else 1), device="cuda", dtype=torch.bfloat16)
    q, s = fp8.act_quant(x, swiglu=swiglu)
    qr, sr = fp8.act_quant_reference(x, swiglu=swiglu)
    got = q.view(torch.float8_e4m3fn).float().view(37, -1, 128) * s.unsqueeze(-1)
    want = qr.view(torch.float8_e4m3fn).float().view(37, -1, 128) * sr.unsqueeze(-1)
    assert torch.allclose(s, sr, rtol=1e-2 if swiglu else 1e-6)
    assert (got - want).abs().max() <= 0.13 * want.abs().max()
    assert ((got - want).abs() < 1e-6).float().mean() > (0.9 if swiglu else 0.999)


def test_act_quant_row_limit(native):
    """Rows at or beyond the device-side limit are left as they were."""
    torch.manual_seed(1)
    x = torch.randn(64, 1024, device="cuda", dtype=torch.bfloat16)
    limit = torch.tensor([0, 23], device="cuda", dtype=torch.int32)
    q = torch.full((64, 512), 7, device="cuda", dtype=torch.uint8)
    s = torch.full((64, 4), -1.0, device="cuda")
    fp8.act_quant(x, swiglu=True, out_q=q, out_s=s, row_limit=limit[1:])
    qr, sr = fp8.act_quant_reference(x, swiglu=True)
    assert torch.allclose(s[:23], sr[:23], rtol=1e-2)
    assert (q[:23] == qr[:23]).float().mean() > 0.9
    assert (q[23:] == 7).all() and (s[23:] == -1.0).all()


@pytest.mark.parametrize("M,Nout,K,splits", [(16, 256, 512, 1), (100, 384, 1024, 1), (200, 256, 2048, 1),
                                              (7, 128, 7168, 4), (64, 7168, 2048, 1)])
def test_dense_fp8_gemm(native, M, Nout, K, splits):
    torch.manual_seed(M + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(Nout, K, device="cuda") * 0.05
    x8, sx = fp8.act_quant(x)
    w8, sw = fp8.quantize_weight(w)
    status = N.new_status("cuda")
    y = fp8.grouped_gemm(x8, sx, fp8.tile_weight(w8), sw, splits=splits, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "fp8 gemm")
    ref = fp8.grouped_gemm_reference(x8, sx, w8, sw)
    err = (y.float() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 1e-2, err


def test_grouped_fp8_gemm_ragged_experts(native, monkeypatch):
    monkeypatch.setenv("ULC_PREFILL_GEMM", "0")        # the weight-stationary kernel at every ring geometry
    torch.manual_seed(3)
    E, Nout, K = 12, 256, 1024
    counts = torch.tensor([0, 3, 17, 1, 0, 130, 16, 64, 2, 0, 300, 5])
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = counts.cumsum(0)
    M = int(offs[-1])
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, Nout, K, device="cuda") * 0.05
    x8, sx = fp8.act_quant(x)
    w8, sw = fp8.quantize_weight(w)
    status = N.new_status("cuda")
    y = fp8.grouped_gemm(x8, sx, fp8.tile_weight(w8), sw, offs.cuda(), status=status)
    y16 = fp8.grouped_gemm(x8, sx, fp8.tile_weight(w8), sw, offs.cuda(), status=status, max_rows=16)
    torch.cuda.synchronize()
    N.raise_on_status(status, "fp8 grouped gemm")
    ref = fp8.grouped_gemm_reference(x8, sx, w8, sw, offs)
    err = (y.float() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 1e-2, err
    # the hint only changes the ring geometry and the fp32 summation order
    assert (y.float() - y16.float()).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-2
    # the list of experts with rows may come ready from the routing kernel
    act = torch.tensor([int((counts > 0).sum())] + [e for e in range(E) if counts[e] > 0] + [0] * int((counts == 0).sum()),
                       dtype=torch.int32, device="cuda")
    ya = fp8.grouped_gemm(x8, sx, fp8.tile_weight(w8), sw, offs.cuda(), status=status, active=act)
    torch.cuda.synchronize()
    assert torch.equal(ya, y)
    for hint in (32, 64):          # every ring geometry, with experts that need several passes
        yh = fp8.grouped_gemm(x8, sx, fp8.tile_weight(w8), sw, offs.cuda(), status=status, max_rows=hint)
        torch.cuda.synchronize()
        N.raise_on_status(status, f"fp8 grouped gemm, hint {hint}")
        assert (yh.float() - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("M", [32, 48, 256])
def test_dense_fp8_gemm_long_k(native, M, monkeypatch):
    """Many K blocks per tile (the ring wraps several times) for each ring geometry."""
    monkeypatch.setenv("ULC_PREFILL_GEMM", "0")
    torch.manual_seed(M)
    Nout, K = 512, 7168
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(Nout, K, device="cuda") * 0.05
    x8, sx = fp8.act_quant(x)
    w8, sw = fp8.quantize_weight(w)
    status = N.new_status("cuda")
    y = fp8.grouped_gemm(x8, sx, fp8.tile_weight(w8), sw, status=status, max_rows=M)
    torch.cuda.synchronize()
    N.raise_on_status(status, "fp8 gemm")
    ref = fp8.grouped_gemm_reference(x8, sx, w8, sw)
    assert (y.float() - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-2


def test_gemm_reduce_scatter_epilogue(native):
    """Row m of the product goes only to peer m // rows_per_peer (every peer buffer is on this GPU)."""
    torch.manual_seed(9)
    M, Nout, K, per = 48, 256, 1024, 16
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(Nout, K, device="cuda") * 0.05
    x8, sx = fp8.act_quant(x)
    w8, sw = fp8.quantize_weight(w)
    wt = fp8.tile_weight(w8)
    status = N.new_status("cuda")
    want = fp8.grouped_gemm(x8, sx, wt, sw, status=status)
    bufs = [torch.zeros(per, Nout, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    fp8.gemm_reduce_scatter(x8, sx, wt, sw, [b.data_ptr() for b in bufs], per, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "gemm reduce-scatter")
    for r in range(3):
        assert torch.equal(bufs[r], want[r * per:(r + 1) * per])


@pytest.mark.parametrize("M,Nout,K,splits", [(32, 2304, 7168, 8), (32, 7168, 16384, 5), (7, 128, 7168, 4),
                                              (16, 512, 2048, 16), (20, 384, 1024, 3)])
def test_dense_split_k_reduced_in_the_kernel(native, M, Nout, K, splits):
    """K splits of a dense decode GEMM: partial tiles meet in the workspace, the last split of each
    tile sums them.  Twice on the same workspace (the tickets reset themselves), also with the result
    sent to 'peer' buffers."""
    torch.manual_seed(M + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(Nout, K, device="cuda") * 0.05
    x8, sx = fp8.act_quant(x)
    w8, sw = fp8.quantize_weight(w)
    wt = fp8.tile_weight(w8)
    status = N.new_status("cuda")
    ref = fp8.grouped_gemm_reference(x8, sx, w8, sw)
    for trial in range(2):
        y = fp8.grouped_gemm(x8, sx, wt, sw, splits=splits, status=status)
        torch.cuda.synchronize()
        N.raise_on_status(status, "fp8 gemm")
        assert (y.float() - ref).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-2
    assert int(fp8.splitk_workspace("cuda")[:4096].view(torch.int32).abs().sum()) == 0
    bufs = [torch.zeros(M, Nout, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    fp8.grouped_gemm(x8, sx, wt, sw, splits=splits, status=status, peer_out=[b.data_ptr() for b in bufs])
    torch.cuda.synchronize()
    N.raise_on_status(status, "fp8 gemm")
    assert torch.equal(bufs[0], y) and torch.equal(bufs[1], y)


@pytest.mark.parametrize("M,Nout,K", [(130, 128, 128), (256, 256, 512), (300, 384, 1024), (1100, 512, 7168),
                                      (2048, 2304, 2048)])
def test_token_major_gemm_dense(native, M, Nout, K):
    """Prefill-sized rows: tokens on the TMEM lanes, one block scale per thread and K block; partial last row tile,
    more items than CTAs, K rings that wrap."""
    torch.manual_seed(M + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(Nout, K, device="cuda") * 0.05
    x8, sx = fp8.act_quant(x)
    w8, sw = fp8.quantize_weight(w)
    status = N.new_status("cuda")
    y = fp8.many_rows_gemm(x8, sx, fp8.tile_weight(w8), sw, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "token-major fp8 gemm")
    ref = fp8.grouped_gemm_reference(x8, sx, w8, sw)
    err = (y.float() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 1e-2, err
    if fp8.many_rows(M, 1):        # the public entry takes the same kernel from these sizes on
        y2 = fp8.grouped_gemm(x8, sx, fp8.tile_weight(w8), sw, status=status)
        torch.cuda.synchronize()
        assert torch.equal(y, y2)


def test_token_major_gemm_ragged_experts(native):
    """Experts with no rows, a few rows, exactly one tile, several tiles; rows behind the last expert stay untouched."""
    torch.manual_seed(5)
    E, Nout, K = 12, 384, 1024
    counts = torch.tensor([0, 3, 128, 1, 0, 130, 16, 64, 257, 0, 300, 5])
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = counts.cumsum(0)
    used = int(offs[-1])
    M = used + 40
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, Nout, K, device="cuda") * 0.05
    x8, sx = fp8.act_quant(x)
    w8, sw = fp8.quantize_weight(w)
    status = N.new_status("cuda")
    out = torch.full((M, Nout), 7.0, device="cuda", dtype=torch.bfloat16)
    y = fp8.many_rows_gemm(x8, sx, fp8.tile_weight(w8), sw, offs.cuda(), out=out, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "token-major grouped fp8 gemm")
    ref = fp8.grouped_gemm_reference(x8[:used], sx[:used], w8, sw, offs)
    err = (y[:used].float() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 1e-2, err
    assert (y[used:] == 7.0).all()
    # against the weight-stationary kernel on the same operands
    import os
    os.environ["ULC_PREFILL_GEMM"] = "0"
    try:
        y0 = fp8.grouped_gemm(x8[:used].contiguous(), sx[:used].contiguous(), fp8.tile_weight(w8), sw, offs.cuda(),
                              status=status)
    finally:
        os.environ.pop("ULC_PREFILL_GEMM")
    torch.cuda.synchronize()
    assert (y[:used].float() - y0.float()).abs().max().item() <= 0.01 * ref.abs().max().item() + 1e-2
