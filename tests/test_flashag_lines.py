"""Wire format of the line all-gather: host model round trip and slab arithmetic (CPU)."""
import numpy as np
import pytest

from ulacache_b200 import flashag


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 31), (7, 300), (30, 64), (31, 5), (64, 257)])
def test_pack_unpack_round_trip(rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    data = rng.standard_normal((rows, cols)).astype(np.float32)
    lens = rng.integers(0, cols + 1, size=rows)
    lens[rng.integers(0, rows)] = cols
    lines = flashag.pack_lines(data, lens, tag=5)
    assert lines.shape[1] == 32 and lines.shape[0] <= flashag.line_count(rows, cols)
    assert (lines[:, 31] == 5).all()
    got, got_len = flashag.unpack_lines(lines, rows, cols, tag=5, fill=-np.inf)
    assert (got_len == lens).all()
    for r in range(rows):
        assert np.array_equal(got[r, : lens[r]], data[r, : lens[r]])
        assert np.isneginf(got[r, lens[r]:]).all()
    with pytest.raises(ValueError):
        flashag.unpack_lines(lines, rows, cols, tag=6, fill=0.0)


def test_line_slab_layout():
    lay = flashag.LineSlabLayout(world=8, max_lines=flashag.line_count(32, 4096), slots=4)
    assert lay.bytes == 4 * 8 * lay.max_lines * 128
    assert lay.line_offset(1, 0) == 8 * lay.max_lines and lay.line_offset(0, 3) == 3 * lay.max_lines
    assert abs(lay.wire_efficiency() - 31 / 32) < 1e-12
    # 32 rows x 4096 columns: two header lines and 4229 payload lines (31 words each)
    assert flashag.line_count(32, 4096) == 2 + (32 * 4096 + 30) // 31
