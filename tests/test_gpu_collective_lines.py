"""Line all-gather kernel on one GPU: the peer is a second slab on the same device whose message
is written by the host model before the launch, so the kernel never waits for another launch."""
import numpy as np
import pytest
import torch

from ulacache_b200 import flashag
from ulacache_b200.ops import _native as N

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,ragged", [(7, 300, True), (32, 4096, False), (64, 257, True), (1, 40, True)])
def test_line_all_gather_against_the_host_model(rows, cols, ragged):
    dev = torch.device("cuda")
    rng = np.random.default_rng(rows + cols)
    world, slots = 2, 2
    max_lines = flashag.line_count(rows, cols)
    words = slots * world * max_lines * 32
    mine = torch.zeros(words, dtype=torch.int32, device=dev)        # my receive slab
    peer = torch.zeros(words, dtype=torch.int32, device=dev)        # the peer's receive slab
    counter = torch.zeros(2, dtype=torch.int32, device=dev)
    status = N.new_status(dev)
    for call in range(1, 4):                                         # three calls: both slots and a reuse
        local = rng.standard_normal((rows, cols)).astype(np.float32)
        other = rng.standard_normal((rows, cols)).astype(np.float32)
        my_len = rng.integers(0, cols + 1, size=rows) if ragged else np.full(rows, cols)
        other_len = rng.integers(0, cols + 1, size=rows) if ragged else np.full(rows, cols)
        slot = (call - 1) % slots
        # the peer's message (rank 1) arrives in my slab before the launch
        msg = flashag.pack_lines(other, other_len, tag=call)
        at = (slot * world + 1) * max_lines * 32
        mine[at: at + msg.size] = torch.from_numpy(msg.reshape(-1).view(np.int32)).to(dev)
        out, out_len = flashag.line_all_gather_raw(
            torch.from_numpy(local).to(dev), torch.from_numpy(my_len.astype(np.int32)).to(dev) if ragged else None,
            [mine.data_ptr(), peer.data_ptr()], 0, world, max_lines, slots, counter, status, fill=-7.0,
            limit_cycles=200_000_000)
        torch.cuda.synchronize()
        N.raise_on_status(status, "line all-gather")
        assert int(counter[0]) == call and int(counter[1]) == 0
        # what I sent is the host model's message, in the peer's slab at [slot][rank 0]
        sent = flashag.pack_lines(local, my_len, tag=call)
        at = (slot * world + 0) * max_lines * 32
        got_sent = peer[at: at + sent.size].cpu().numpy().view(np.uint32).reshape(-1, 32)
        assert np.array_equal(got_sent, sent)
        # what I received
        want0 = np.full((rows, cols), -7.0, np.float32)
        want1 = np.full((rows, cols), -7.0, np.float32)
        for r in range(rows):
            want0[r, : my_len[r]] = local[r, : my_len[r]]
            want1[r, : other_len[r]] = other[r, : other_len[r]]
        assert np.array_equal(out[0].cpu().numpy(), want0)
        assert np.array_equal(out[1].cpu().numpy(), want1)
        assert np.array_equal(out_len.cpu().numpy(), np.stack([my_len, other_len]).astype(np.int32))


def test_line_all_gather_reports_a_missing_message():
    """Nothing ever writes the peer's lines: the bounded wait runs out, the status word says so and the
    context stays usable (the missing rows come back as the fill value)."""
    dev = torch.device("cuda")
    rows, cols, world, slots = 4, 64, 2, 2
    max_lines = flashag.line_count(rows, cols)
    mine = torch.zeros(slots * world * max_lines * 32, dtype=torch.int32, device=dev)
    peer = torch.zeros_like(mine)
    counter = torch.zeros(2, dtype=torch.int32, device=dev)
    status = N.new_status(dev)
    local = torch.randn(rows, cols, device=dev)
    out, _ = flashag.line_all_gather_raw(local, None, [mine.data_ptr(), peer.data_ptr()], 0, world, max_lines, slots,
                                         counter, status, fill=-1.0, limit_cycles=2_000_000)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        N.raise_on_status(status, "line all-gather")
    assert torch.equal(out[0], local) and bool((out[1] == -1.0).all())
    assert float(torch.ones(4, device=dev).sum()) == 4.0
