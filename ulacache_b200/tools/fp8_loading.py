"""Block-scale helpers for loading fp8 checkpoints.

Reference: ulacache/tools/fp8_loading.py:1-36 (block-scale dequant helper).
"""
from __future__ import annotations


def dequantize_block_scaled(q, scale, block: int = 128):
    """``q`` float8_e4m3fn (or its uint8 bytes) [..., N, K], ``scale`` fp32 [..., ceil(N/block), ceil(K/block)]
    -> fp32 [..., N, K]."""
    import torch

    if q.dtype == torch.uint8:
        q = q.view(torch.float8_e4m3fn)
    n, k = q.shape[-2], q.shape[-1]
    s = scale.repeat_interleave(block, dim=-2)[..., :n, :].repeat_interleave(block, dim=-1)[..., :k]
    return q.float() * s


def requantize_for_kernels(weight_fp32):
    """fp32 [N, K] (N, K multiples of 128) -> (tile-major fp8 bytes, block scales) as the grouped GEMM reads them."""
    from ..ops import fp8

    q, s = fp8.quantize_weight(weight_fp32)
    return fp8.tile_weight(q), s


def aligned_row_block_scales(values, scales, block_size) -> bool:
    """Whether ``scales`` are fp32 ROW-block scales of ``values`` [rows, cols]: ``block_size`` = (1, width), ``cols`` a
    multiple of ``width`` and ``scales`` [rows, cols / width] on the same device (the layout activation and KV
    quantisers produce, as opposed to the 128 x 128 blocks of weights)."""
    import torch

    if (len(block_size) != 2 or block_size[0] != 1 or block_size[1] <= 0 or values.ndim != 2 or scales.ndim != 2
            or scales.dtype != torch.float32):
        return False
    rows, cols = values.shape
    width = block_size[1]
    return (rows > 0 and cols > 0 and cols % width == 0 and tuple(scales.shape) == (rows, cols // width)
            and scales.device == values.device)


def dequantize_aligned_rows(values, scales, block_size):
    """fp32 copy of ``values`` with every row block multiplied by its scale in ONE batched multiply (no loop over
    blocks).  Raises when the scales are not aligned row blocks.

    Reference: ulacache/tools/fp8_loading.py:4-36."""
    import torch

    if not aligned_row_block_scales(values, scales, block_size):
        raise ValueError("expected fp32 scales over aligned row blocks")
    if values.dtype == torch.uint8:
        values = values.view(torch.float8_e4m3fn)
    rows, cols = values.shape
    width = block_size[1]
    out = values.to(torch.float32)
    out.view(rows, cols // width, width).mul_(scales.unsqueeze(-1))
    return out
