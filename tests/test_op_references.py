"""CPU reference forms of the kernel wrappers (what every GPU numerics test compares against)
agree with plain PyTorch arithmetic on small cases."""
import torch

from ulacache_b200.ops import fp8, topk


def test_act_quant_reference_roundtrip_and_row_limit():
    torch.manual_seed(0)
    x = torch.randn(12, 256).to(torch.bfloat16)
    q, s = fp8.act_quant(x)                                   # CPU tensors take the reference path
    back = q.view(torch.float8_e4m3fn).float().view(12, 2, 128) * s.unsqueeze(-1)
    assert (back.view(12, 256) - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    # SwiGLU form: [gate | up] -> silu(gate) * up
    y = torch.randn(12, 512).to(torch.bfloat16)
    q2, s2 = fp8.act_quant(y, swiglu=True)
    want = torch.nn.functional.silu(y[:, :256].float()) * y[:, 256:].float()
    back2 = (q2.view(torch.float8_e4m3fn).float().view(12, 2, 128) * s2.unsqueeze(-1)).view(12, 256)
    assert (back2 - want).abs().max() <= 0.08 * want.abs().max() + 1e-3
    # rows at or beyond the limit are cleared by the reference (left untouched by the kernel)
    q3, s3 = fp8.act_quant(y, swiglu=True, row_limit=torch.tensor([5], dtype=torch.int32))
    assert torch.equal(q3[:5], q2[:5]) and torch.equal(s3[:5], s2[:5])
    assert int(q3[5:].abs().sum()) == 0 and float(s3[5:].abs().sum()) == 0.0


def test_topk_reference_lengths_ties_and_tables():
    s = torch.tensor([[0.5, 3.0, 3.0, 1.0, 3.0, -1.0], [9.0, 8.0, 7.0, 6.0, 5.0, 4.0]])
    out = topk.topk(s, 2)                                     # ties at the k-th value: lowest positions win
    assert sorted(out[0].tolist()) == [1, 2] and sorted(out[1].tolist()) == [0, 1]
    out = topk.topk(s, 4, lengths=torch.tensor([3, 2], dtype=torch.int32))
    assert sorted(out[0].tolist()) == sorted([0, 1, 2, -1])      # three valid scores, padded with -1
    assert sorted(out[1].tolist()) == sorted([0, 1, -1, -1])
    table = (torch.arange(6, dtype=torch.int32) * 10).repeat(2, 1)
    out = topk.topk(s, 2, xform=table)
    assert sorted(out[0].tolist()) == [10, 20]


def test_pick_splits_prefers_full_rounds():
    # 56 feature tiles x 128 K blocks (o_proj): 2 splits = 112 items in ONE round of 148 CTAs; the
    # per-item cost makes this beat 5 splits (280 items, two rounds), as measured at 32 rows
    assert fp8.pick_splits(7168, 16384) == 2
    # 18 feature tiles (the fused input projection): split until one round is nearly full
    assert fp8.pick_splits(2304, 7168) * 18 <= 148
    # enough tiles for every SM: no split
    assert fp8.pick_splits(32768, 1536) == 1
    assert 1 <= fp8.pick_splits(2304, 7168) <= 16


def test_shared_expert_placement_rule():
    """The sort kernel's rule for where the shared expert's items start (host copy of the device
    function): its CTAs must be ones that the round-robin deal gives no extra item."""
    from ulacache_b200.ops import glue

    for n_routed, tiles, grid in [(32, 32, 148), (32, 56, 148), (256, 32, 148), (16, 32, 148), (7, 56, 132)]:
        p = glue.shared_expert_position(n_routed, tiles, grid)
        assert 0 <= p <= n_routed
        items = (n_routed + 1) * tiles
        rem = items % grid
        if p < n_routed:                      # a placement was found: check the property
            start = (p * tiles) % grid
            assert start >= rem and start + tiles <= grid
            assert all(((q * tiles) % grid) < rem or ((q * tiles) % grid) + tiles > grid for q in range(p))
    assert glue.shared_expert_position(32, 32, 148) == 1 and glue.shared_expert_position(32, 56, 148) == 4
    assert glue.shared_expert_position(31, 32, 148) == 31          # no position qualifies: last
    assert glue.shared_expert_position(32, 0, 148) == 32           # rule switched off
