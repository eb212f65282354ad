"""Fused gather + sparse MLA decode attention against the fp32 PyTorch reference."""
import pytest
import torch

from ulacache_b200.ops import _native as N
from ulacache_b200.ops import records, sparse_mla
from ulacache_b200.storage import layout as L

pytestmark = pytest.mark.gpu


def _pool(slots, fmt="mla.scaled656.fp8.v1", seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    latent = torch.randn(slots, 512, device="cuda", generator=g)
    rope = torch.randn(slots, 64, device="cuda", generator=g)
    return records.ENCODERS[fmt](latent, rope).contiguous()


def _view(pool):
    dummy_dir = torch.zeros(1, dtype=torch.int32, device="cuda")
    return records.make_pool_view(hbm_ptrs=[pool.data_ptr()], dir_ptrs=[dummy_dir.data_ptr()], host_ptr=0,
                                  dir_len=1, hbm_slots=pool.shape[0], host_slots=0, rec_bytes=pool.shape[1],
                                  owners=L.OwnerMap(1, 6), my_rank=0), dummy_dir


@pytest.mark.parametrize("B,H,K,splits,masked", [
    (2, 64, 64, 1, False), (3, 16, 256, 1, True), (2, 128, 512, 1, True), (1, 128, 2048, 4, True),
    (5, 16, 2048, 2, False), (4, 64, 192, 3, True)])
def test_sparse_mla_matches_reference(native, B, H, K, splits, masked):
    torch.manual_seed(B * 1000 + K)
    slots = 8192
    pool = _pool(slots)
    view, keep = _view(pool)
    q = (torch.randn(B, H, 576, device="cuda") * 0.5).to(torch.bfloat16)
    loc = torch.stack([torch.randperm(slots, device="cuda")[:K] for _ in range(B)]).to(torch.int32)
    if masked:
        loc[torch.rand(B, K, device="cuda") < 0.2] = -1
        loc[0, K // 2:] = -1
    status = N.new_status("cuda")
    scale = 576 ** -0.5
    out, lse = sparse_mla.sparse_mla_decode(view, q, loc, scale, splits=splits, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "sparse_mla")
    ref_o, ref_l = sparse_mla.sparse_mla_reference(q, [pool], loc, scale)
    assert torch.allclose(lse, ref_l, atol=2e-2, rtol=1e-3), (lse - ref_l).abs().max()
    err = (out.float() - ref_o).abs().max().item()
    assert err < 2e-2, err


def test_sparse_mla_lens_and_bf16_records(native):
    torch.manual_seed(7)
    fmt = "mla.bf16.1152.v1"
    pool = _pool(4096, fmt)
    view, keep = _view(pool)
    B, H, K = 3, 32, 320
    q = (torch.randn(B, H, 576, device="cuda") * 0.5).to(torch.bfloat16)
    loc = torch.stack([torch.randperm(4096, device="cuda")[:K] for _ in range(B)]).to(torch.int32)
    lens = torch.tensor([320, 100, 0], dtype=torch.int32, device="cuda")
    status = N.new_status("cuda")
    out, lse = sparse_mla.sparse_mla_decode(view, q, loc, 0.05, lens=lens, splits=1, fmt_code=2, status=status)
    torch.cuda.synchronize()
    N.raise_on_status(status, "sparse_mla")
    ref_o, ref_l = sparse_mla.sparse_mla_reference(q, [pool], loc, 0.05, decode=records.decode_bf16, lens=lens)
    assert torch.allclose(out.float(), ref_o, atol=2e-2)
    assert torch.isinf(lse[2]).all() and (out[2] == 0).all()
    assert torch.allclose(lse[:2], ref_l[:2], atol=2e-2)


def test_cta_pair_launch_matches_independent_ctas(native):
    """The two-CTA cluster variant (each CTA gathers half of every tile into both) gives the results of
    the default launch, with masked tokens, KV splits and both record formats' common path."""
    from ulacache_b200.ops import sparse_mla as M

    torch.manual_seed(7)
    slots = 8192
    pool = _pool(slots)
    view, keep = _view(pool)
    status = N.new_status("cuda")
    for B, K, splits in ((3, 2048, 2), (2, 700, 1), (1, 64, 1)):
        q = (torch.randn(B, 128, 576, device="cuda") * 0.5).to(torch.bfloat16)
        loc = torch.stack([torch.randperm(slots, device="cuda")[:K] for _ in range(B)]).to(torch.int32)
        loc[torch.rand(B, K, device="cuda") < 0.15] = -1
        outs = []
        for pair in (False, True):
            M.set_pair_launch(pair)
            try:
                o, lse = M.sparse_mla_decode(view, q, loc, 576 ** -0.5, splits=splits, status=status)
                torch.cuda.synchronize()
            finally:
                M.set_pair_launch(False)
            N.raise_on_status(status, "sparse_mla pair")
            outs.append((o.float(), lse))
        assert torch.allclose(outs[0][0], outs[1][0], atol=2e-3, rtol=2e-2)
        assert torch.allclose(outs[0][1], outs[1][1], atol=1e-3, rtol=1e-3)
