"""Block-scaled fp8 linear algebra: quantisers, the grouped GEMM launcher and references.

Weights are fp8 e4m3 with one fp32 scale per 128 x 128 block; activations are fp8
with one scale per token per 128 columns (the DeepSeek-V3 recipe).
"""
from __future__ import annotations

import ctypes as C

from . import _native as N
from .records import FP8_MAX, SCALE_FLOOR, _exact_div


def quantize_weight(w):
    """[..., Nout, K] float -> (uint8 fp8 [..., Nout, K], fp32 scales [..., Nout/128, K/128])."""
    import torch

    *lead, n, k = w.shape
    assert n % 128 == 0 and k % 128 == 0
    blocks = w.float().reshape(*lead, n // 128, 128, k // 128, 128)
    amax = blocks.abs().amax(dim=(-3, -1))
    scale = _exact_div(torch.clamp(amax, min=SCALE_FLOOR), FP8_MAX)
    q = (blocks / scale.unsqueeze(-1).unsqueeze(-3)).to(torch.float8_e4m3fn)
    return q.reshape(*lead, n, k).view(torch.uint8).contiguous(), scale.contiguous()


def random_fp8_weight(shape, *, device, std=0.02, generator=None, tiled=True):
    """Random-init block-scaled weight without materialising an fp32 copy larger than one
    chunk: uniform random fp8 codes with a constant block scale chosen for ``std``.
    ``shape`` is the canonical [..., Nout, K]; with ``tiled`` the bytes come back in the
    kernel's tile-major layout [..., Nout/128, K/128, 128, 128]."""
    import torch

    *lead, n, k = shape
    if tiled:
        shape = (*lead, n // 128, k // 128, 128, 128)
    q = torch.empty(shape, dtype=torch.uint8, device=device)
    flat = q.view(-1)
    chunk = 1 << 28
    for i in range(0, flat.numel(), chunk):
        part = flat[i:i + chunk]
        part.random_(0, 256, generator=generator)
    # clear NaN codes (0x7f / 0xff) and keep magnitudes moderate: mask to exponent <= 7
    q.bitwise_and_(0xBF)
    # values are roughly uniform in log-magnitude up to 1.875; rms about 0.6
    scale = torch.full((*lead, n // 128, k // 128), std / 0.6, dtype=torch.float32, device=device)
    return q, scale


def tile_weight(q):
    """Canonical [..., Nout, K] fp8 bytes -> tile-major [..., Nout/128, K/128, 128, 128], the layout
    the GEMM kernel streams (each 128 x 128 block contiguous)."""
    *lead, n, k = q.shape
    return q.reshape(*lead, n // 128, 128, k // 128, 128).transpose(-3, -2).contiguous()


def untile_weight(t):
    *lead, nt, kt, a, b = t.shape
    return t.transpose(-3, -2).reshape(*lead, nt * 128, kt * 128)


def dequantize_weight(q, scale):
    import torch

    *lead, n, k = q.shape
    w = q.view(torch.float8_e4m3fn).float().reshape(*lead, n // 128, 128, k // 128, 128)
    return (w * scale.unsqueeze(-1).unsqueeze(-3)).reshape(*lead, n, k)


def act_quant_reference(x, *, swiglu=False):
    import torch

    xf = x.float()
    if swiglu:
        k = xf.shape[1] // 2
        xf = torch.nn.functional.silu(xf[:, :k]) * xf[:, k:]
    m, k = xf.shape
    g = xf.view(m, k // 128, 128)
    amax = g.abs().amax(dim=-1)
    scale = _exact_div(torch.clamp(amax, min=SCALE_FLOOR), FP8_MAX)
    q = (g * (1.0 / scale).unsqueeze(-1)).to(torch.float8_e4m3fn).view(m, k)
    return q.view(torch.uint8), scale


def act_quant(x, *, swiglu=False, out_q=None, out_s=None, row_limit=None):
    """bf16 [M, K] (or [M, 2K] gate|up with ``swiglu``) -> (uint8 fp8 [M, K], fp32 [M, K/128]).
    ``row_limit``: int32 device tensor (first element used); rows at or beyond it are left untouched
    (for buffers sized for the worst case of a routing step, of which only the head is filled)."""
    import torch

    if not x.is_cuda:
        q, s = act_quant_reference(x, swiglu=swiglu)
        if row_limit is not None:
            n = int(row_limit.reshape(-1)[0])
            q[n:] = 0
            s[n:] = 0
        return q, s
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    m = x.shape[0]
    k = x.shape[1] // 2 if swiglu else x.shape[1]
    if out_q is None:
        out_q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    if out_s is None:
        out_s = torch.empty((m, k // 128), dtype=torch.float32, device=x.device)
    N.check(N.cuda().ulc_act_quant_rows(N.ptr(x), C.c_longlong(x.stride(0)), N.ptr(out_q), N.ptr(out_s), C.c_int(m),
                                        C.c_int(k), C.c_int(1 if swiglu else 0), N.ptr(row_limit), N.stream()),
            "act_quant")
    return out_q, out_s


def grouped_gemm_reference(x8, sx, w8, sw, offs=None):
    """fp32 reference with exact block scaling (``w8`` canonical or tile-major).  Returns fp32 [M, Nout]."""
    import torch

    if w8.dim() >= 4:
        w8 = untile_weight(w8)
    m, k = x8.shape
    xf = (x8.view(torch.float8_e4m3fn).float().view(m, k // 128, 128) * sx.unsqueeze(-1)).view(m, k)
    if w8.dim() == 2:
        w8, sw = w8.unsqueeze(0), sw.unsqueeze(0)
    wf = dequantize_weight(w8, sw)
    e = wf.shape[0]
    out = torch.zeros((m, wf.shape[1]), dtype=torch.float32, device=x8.device)
    bounds = [0, m] if offs is None else offs.tolist()
    for i in range(e):
        a, b = bounds[i], bounds[i + 1]
        if b > a:
            out[a:b] = xf[a:b] @ wf[i].t()
    return out


_SPLITK_WS = {}
SPLITK_WS_BYTES = 24 << 20


def splitk_workspace(device):
    """Per-device scratch of the in-kernel split-K reduction (partial tiles + tickets), zero when
    created; every GEMM leaves it ready for the next.  GEMMs that use it must be ordered on one
    stream.  Create it (one GEMM call, or this function) before capturing a CUDA graph."""
    import torch

    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _SPLITK_WS:
        _SPLITK_WS[key] = torch.zeros(SPLITK_WS_BYTES, dtype=torch.uint8, device=device)
    return _SPLITK_WS[key]


def _splitk_fits(m, nout, splits, max_rows):
    if 0 < max_rows < m:          # several passes over the rows: the partial tiles of one pass would be overwritten
        return False
    return m <= 32 and nout // 128 <= 1024 and 4096 + (nout // 128) * splits * 32 * 128 * 4 <= SPLITK_WS_BYTES


def grouped_gemm(x8, sx, w8, sw, offs=None, *, splits=1, out=None, status=None, work=None, max_rows=0,
                 peer_out=None, active=None, peer_rows=0):
    """``y[m] = x[m] @ w[expert(m)]^T`` with block scales.  ``w8`` is TILE-MAJOR
    ([E,] Nout/128, K/128, 128, 128; see ``tile_weight``); ``offs`` int32 [E+1] gives each
    expert's row range (rows sorted by expert); ``max_rows`` bounds the rows of one expert
    (performance hint).  ``peer_out``: list of device addresses of bf16 [M, Nout] buffers (peer
    GPUs' receive slots) that get the result instead of a returned tensor (needs splits == 1).
    ``active``: int32 [E + 1] = [number of experts with rows, their ids ascending] when the routing
    kernel already produced it (``ops.glue.moe_sort``).  Returns bf16 [M, Nout] (None with ``peer_out``)."""
    import torch

    if not x8.is_cuda:
        return grouped_gemm_reference(x8, sx, w8, sw, offs).to(torch.bfloat16)
    if w8.dim() == 4:
        w8, sw = w8.unsqueeze(0), sw.unsqueeze(0)
    assert w8.dim() == 5 and w8.shape[-1] == 128 and w8.shape[-2] == 128, "weights must be tile-major"
    e, nout, k = w8.shape[0], w8.shape[1] * 128, w8.shape[2] * 128
    m = x8.shape[0]
    assert x8.is_contiguous() and w8.is_contiguous() and sx.is_contiguous() and sw.is_contiguous()
    if not peer_out and many_rows(m, e, max_rows):
        if out is None:
            out = torch.empty((m, nout), dtype=torch.bfloat16, device=x8.device)
        return many_rows_gemm(x8, sx, w8, sw, offs, out=out, status=status)
    if splits > 1 and e == 1 and _splitk_fits(m, nout, splits, max_rows):
        # dense layer at decode size: K splits reduced inside the kernel (no cleared fp32 buffer, no
        # atomics, no conversion launch); the result may also go straight to peers
        ws = splitk_workspace(x8.device)
        if out is None and not peer_out:
            out = torch.empty((m, nout), dtype=torch.bfloat16, device=x8.device)
        n = len(peer_out) if peer_out else 0
        arr = (C.c_void_p * max(n, 1))(*(peer_out or [0]))
        N.check(N.cuda().ulc_fp8_gemm_splitk(
            N.ptr(x8), N.ptr(sx), N.ptr(w8), N.ptr(sw), C.c_int(m), C.c_int(nout), C.c_int(k), C.c_int(splits),
            C.c_int(max_rows), N.ptr(out), arr, C.c_int(n), C.c_int(peer_rows), N.ptr(ws), C.c_longlong(ws.numel()),
            N.ptr(status), N.stream()), "fp8_grouped_gemm")
        return out
    if peer_out:
        splits = 1
        if e > 1 and work is None:
            work = torch.empty(e + 1, dtype=torch.int32, device=x8.device)
        arr = (C.c_void_p * len(peer_out))(*peer_out)
        N.check(N.cuda().ulc_fp8_grouped_gemm_peers(
            N.ptr(x8), N.ptr(sx), N.ptr(w8), N.ptr(sw), N.ptr(offs), C.c_int(m), C.c_int(nout), C.c_int(k), C.c_int(e),
            C.c_int(1), C.c_int(max_rows), C.c_void_p(0), arr, C.c_int(len(peer_out)), N.ptr(work), N.ptr(status),
            N.stream()), "fp8_grouped_gemm" if e == 1 else "fp8_grouped_gemm_experts")
        return None
    if splits > 1:
        acc = torch.zeros((m, nout), dtype=torch.float32, device=x8.device)
        target = acc
    else:
        if out is None:
            out = torch.empty((m, nout), dtype=torch.bfloat16, device=x8.device)
        target = out
    if e > 1 and active is not None and splits == 1:
        # the routing sort already left [count, active expert ids] on the device
        N.check(N.cuda().ulc_fp8_grouped_gemm_prepared(N.ptr(x8), N.ptr(sx), N.ptr(w8), N.ptr(sw), N.ptr(offs), C.c_int(m),
                                                       C.c_int(nout), C.c_int(k), C.c_int(e), C.c_int(max_rows),
                                                       N.ptr(target), N.ptr(active), N.ptr(status), N.stream()),
                "fp8_grouped_gemm_experts")
        return out
    if e > 1 and work is None:
        work = torch.empty(e + 1, dtype=torch.int32, device=x8.device)
    N.check(N.cuda().ulc_fp8_grouped_gemm(N.ptr(x8), N.ptr(sx), N.ptr(w8), N.ptr(sw), N.ptr(offs), C.c_int(m),
                                          C.c_int(nout), C.c_int(k), C.c_int(e), C.c_int(splits), C.c_int(max_rows),
                                          N.ptr(target), N.ptr(work), N.ptr(status), N.stream()),
            "fp8_grouped_gemm" if e == 1 else "fp8_grouped_gemm_experts")
    if splits > 1:
        if out is None:
            return acc.to(torch.bfloat16)
        out.copy_(acc)
    return out


MANY_ROWS_DENSE = 512          # token rows from which a dense layer takes the token-major kernel
MANY_ROWS_PER_EXPERT = 32      # expected rows per expert from which a grouped layer does


def many_rows(m: int, experts: int, max_rows: int = 0) -> bool:
    """Whether a GEMM of ``m`` token rows over ``experts`` weight sets is prefill-sized: the weight-stationary
    decode kernel re-streams every weight tile once per 128 rows and pays a column-scaled epilogue; from these
    sizes on the token-major kernel (``csrc/fp8_prefill_gemm.cu``) wins.  ``m`` of a grouped layer counts every
    allocated row (other ranks' experts included), so the caller's expected rows per expert (``max_rows``, the ring
    geometry hint: 64 means more than 24 expected) decides when given.  ``ULC_PREFILL_GEMM=0`` switches it off."""
    import os

    if os.environ.get("ULC_PREFILL_GEMM", "1") == "0" or m < 256:
        return False
    if experts == 1:
        return m >= MANY_ROWS_DENSE
    if max_rows > 0:
        return max_rows >= 64
    return m >= MANY_ROWS_PER_EXPERT * experts


def many_rows_gemm(x8, sx, w8, sw, offs=None, *, out=None, status=None):
    """Token-major block-scaled fp8 GEMM (tokens on the TMEM lanes, one scale per thread and K block).  Same
    operands as ``grouped_gemm``; ``w8`` [E, Nout/128, K/128, 128, 128].  Returns bf16 [M, Nout]."""
    import torch

    if w8.dim() == 4:
        w8, sw = w8.unsqueeze(0), sw.unsqueeze(0)
    e, nout, k = w8.shape[0], w8.shape[1] * 128, w8.shape[2] * 128
    m = x8.shape[0]
    if out is None:
        out = torch.empty((m, nout), dtype=torch.bfloat16, device=x8.device)
    assert out.is_contiguous() and out.shape == (m, nout)
    N.check(N.cuda().ulc_fp8_prefill_gemm(
        N.ptr(x8), N.ptr(sx), N.ptr(w8), N.ptr(sw), N.ptr(offs),
        C.c_int(m), C.c_int(nout), C.c_int(k), C.c_int(e), C.c_int((m + 127) // 128 + e), N.ptr(out), N.ptr(status),
        N.stream()), "fp8_prefill_gemm")
    return out


def pick_splits(nout: int, k: int, experts: int = 1, sm_count: int = 148) -> int:
    """K splits of a dense weight-streaming GEMM.  The persistent kernel deals items
    (n-tile, K split) round robin to ``sm_count`` CTAs, so the cost of a choice is
    rounds * (bytes of one item / per-SM bandwidth + per-item overhead); more splits also pay for
    clearing and converting the fp32 accumulation buffer."""
    tiles = (nout // 128) * experts
    kb = k // 128
    if kb < 1 or nout < 128:
        raise ValueError("fp8 block-scaled GEMMs need at least one 128 x 128 block")
    if tiles >= sm_count:
        return 1
    best, best_cost = 1, None
    for s in range(1, min(16, max(1, kb // 4)) + 1):
        per = (kb + s - 1) // s
        items = tiles * ((kb + per - 1) // per)
        rounds = (items + sm_count - 1) // sm_count
        # microseconds: a K block streams in 0.37 us at one SM's share of the HBM bandwidth; an item
        # costs about 4 us of pipeline fill and epilogue drain; the in-kernel reduction reads one more
        # partial tile per split (measured on the decode projections at 32 rows)
        cost = rounds * (per * 16384 / 44000.0 + 4.0) + (0.5 * s if s > 1 else 0.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def gemm_reduce_scatter(x8, sx, w8, sw, peer_out, rows_per_peer, *, status=None):
    """``y = x @ w^T`` whose row m is stored (bf16) only to ``peer_out[m // rows_per_peer]`` at row
    ``m % rows_per_peer``: the send half of a reduce-scatter runs in the GEMM epilogue.  ``w8``
    tile-major [Nout/128, K/128, 128, 128]; ``peer_out`` device addresses of bf16
    [rows_per_peer, Nout] receive blocks (one per rank, this rank included)."""
    assert x8.is_cuda and w8.dim() == 4
    nout, k = w8.shape[0] * 128, w8.shape[1] * 128
    arr = (C.c_void_p * len(peer_out))(*peer_out)
    N.check(N.cuda().ulc_fp8_gemm_reduce_scatter(N.ptr(x8), N.ptr(sx), N.ptr(w8), N.ptr(sw), C.c_int(x8.shape[0]),
                                                 C.c_int(nout), C.c_int(k), C.c_int(rows_per_peer), arr,
                                                 C.c_int(len(peer_out)), N.ptr(status), N.stream()),
            "fp8_gemm_reduce_scatter")
