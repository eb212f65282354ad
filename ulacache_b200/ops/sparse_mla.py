"""Sparse MLA decode attention fused with the KV gather: launcher and reference.

The kernel (``csrc/sparse_mla.cu``) reads the selected records straight from the
owners' pools (local HBM or peer HBM over NVLink) named by ``loc`` and runs
QK^T / PV on the tcgen05 tensor cores.  ``sparse_mla_reference`` is the fp32
PyTorch statement of the same computation.
"""
from __future__ import annotations

import ctypes as C

from . import _native as N
from . import records


def sparse_mla_reference(q, planes, loc, sm_scale, *, decode=records.decode_scaled656, lens=None):
    """q [B,H,576]; planes: list (per owner rank) of uint8 [slots, record_bytes]; loc int32 [B,K]
    (rank << 28 | slot, -1 masked).  Returns (out fp32 [B,H,512], lse fp32 [B,H])."""
    import torch

    B, H, _ = q.shape
    K = loc.shape[1]
    out = torch.zeros(B, H, 512, dtype=torch.float32, device=q.device)
    lse = torch.full((B, H), float("-inf"), dtype=torch.float32, device=q.device)
    qf = q.float()
    for b in range(B):
        l = loc[b]
        if lens is not None:
            l = l[: int(lens[b])]
        valid = l >= 0
        if not bool(valid.any()):
            continue
        lv = l[valid]
        rank, slot = (lv >> 28) & 7, (lv & 0x0FFFFFFF).long()
        rows = torch.empty((lv.numel(), planes[0].shape[-1]), dtype=torch.uint8, device=q.device)
        for r in range(len(planes)):
            m = rank == r
            if bool(m.any()):
                rows[m] = planes[r][slot[m]]
        kv = decode(rows)                      # [n, 576]
        s = qf[b] @ kv.t() * sm_scale          # [H, n]
        lse[b] = torch.logsumexp(s, dim=-1)
        out[b] = torch.softmax(s, dim=-1) @ kv[:, :512]
    return out, lse


def set_pair_launch(on: bool):
    """``True``: the two head blocks of a (query, KV split) run as a cluster of two CTAs that share every K
    tile (each gathers half of it into both CTAs' shared memory).  Measured 7 % slower than independent
    CTAs (the default), see ``csrc/sparse_mla.cu``; kept for comparisons (``ULC_MLA_PAIR=1``)."""
    N.cuda().ulc_sparse_mla_set_pair(C.c_int(int(on)))


_pair_env_applied = False


def _apply_pair_env():
    global _pair_env_applied
    if not _pair_env_applied:
        import os

        _pair_env_applied = True
        if os.environ.get("ULC_MLA_PAIR", "0") == "1":
            set_pair_launch(True)


def default_splits(B: int, H: int, K: int, sm_count: int = 148) -> int:
    """KV splits so that at least one wave of CTAs exists at small batch."""
    ctas = B * ((H + 63) // 64)
    if ctas >= sm_count:
        return 1
    max_splits = max(1, K // 256)
    return max(1, min(max_splits, sm_count // max(ctas, 1)))


def scratch_bytes(B: int, H: int, splits: int) -> int:
    return 0 if splits <= 1 else splits * B * H * 513 * 4


def sparse_mla_decode(pool_view, q, loc, sm_scale, *, lens=None, splits=0, fmt_code=0, out=None, lse=None,
                      scratch=None, status=None):
    """Launch the fused gather + attention kernel.  ``q`` bf16 [B,H,576] contiguous,
    ``loc`` int32 [B,K].  Returns (out bf16 [B,H,512], lse fp32 [B,H])."""
    import torch

    assert q.is_cuda and q.dtype == torch.bfloat16 and q.is_contiguous() and q.shape[-1] == 576
    assert loc.dtype == torch.int32 and loc.stride(1) == 1
    _apply_pair_env()
    B, H, _ = q.shape
    K = loc.shape[1]
    if splits <= 0:
        splits = default_splits(B, H, K)
    if out is None:
        out = torch.empty((B, H, 512), dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty((B, H), dtype=torch.float32, device=q.device)
    if splits > 1 and scratch is None:
        scratch = torch.empty(scratch_bytes(B, H, splits), dtype=torch.uint8, device=q.device)
    code = N.cuda().ulc_sparse_mla_decode(
        C.byref(pool_view), N.ptr(q), N.ptr(loc), C.c_longlong(loc.stride(0)), N.ptr(lens), C.c_int(B),
        C.c_int(H), C.c_int(K), C.c_float(sm_scale), C.c_int(fmt_code), C.c_int(splits), N.ptr(out),
        N.ptr(lse), N.ptr(scratch), N.ptr(status), N.stream())
    N.check(code, "sparse_mla_decode")
    return out, lse


def sparse_mla_decode_strided(pool_view, q_lat, q_rope, loc, sm_scale, *, out, lens=None, fmt_code=0, lse=None,
                              status=None):
    """Strided form without KV splits.  ``q_lat`` bf16 [..] viewed as [B,H,512] with arbitrary (8-element
    aligned) strides over B and H (e.g. the [H,B,512] result of a head-batched GEMM, transposed view),
    ``q_rope`` likewise [B,H,64]; ``out`` bf16 viewed [B,H,512] with arbitrary strides."""
    import torch

    B, H, _ = q_lat.shape
    assert q_lat.stride(2) == 1 and q_rope.stride(2) == 1 and out.stride(2) == 1
    code = N.cuda().ulc_sparse_mla_decode_ex(
        C.byref(pool_view), N.ptr(q_lat), C.c_longlong(q_lat.stride(0)), C.c_longlong(q_lat.stride(1)),
        N.ptr(q_rope), C.c_longlong(q_rope.stride(0)), C.c_longlong(q_rope.stride(1)), N.ptr(loc),
        C.c_longlong(loc.stride(0)), N.ptr(lens), C.c_int(B), C.c_int(H), C.c_int(loc.shape[1]),
        C.c_float(sm_scale), C.c_int(fmt_code), C.c_int(1), N.ptr(out), C.c_longlong(out.stride(0)),
        C.c_longlong(out.stride(1)), N.ptr(lse), C.c_void_p(0), N.ptr(status), N.stream())
    N.check(code, "sparse_mla_decode")
    return out


def sparse_mla_decode_strided_auto(pool_view, q_lat, q_rope, loc, sm_scale, *, fmt_code=0, lens=None, status=None,
                                   splits=0):
    """Strided queries, dense output ``[B,H,512]`` (so KV splits can be used at small batch).
    Returns (out bf16 [B,H,512], lse fp32 [B,H])."""
    import torch

    _apply_pair_env()
    B, H, _ = q_lat.shape
    K = loc.shape[1]
    if splits <= 0:
        splits = default_splits(B, H, K)
    out = torch.empty((B, H, 512), dtype=torch.bfloat16, device=q_lat.device)
    lse = torch.empty((B, H), dtype=torch.float32, device=q_lat.device)
    scratch = torch.empty(scratch_bytes(B, H, splits), dtype=torch.uint8, device=q_lat.device) if splits > 1 else None
    code = N.cuda().ulc_sparse_mla_decode_ex(
        C.byref(pool_view), N.ptr(q_lat), C.c_longlong(q_lat.stride(0)), C.c_longlong(q_lat.stride(1)),
        N.ptr(q_rope), C.c_longlong(q_rope.stride(0)), C.c_longlong(q_rope.stride(1)), N.ptr(loc),
        C.c_longlong(loc.stride(0)), N.ptr(lens), C.c_int(B), C.c_int(H), C.c_int(K), C.c_float(sm_scale),
        C.c_int(fmt_code), C.c_int(splits), N.ptr(out), C.c_longlong(H * 512), C.c_longlong(512), N.ptr(lse),
        N.ptr(scratch), N.ptr(status), N.stream())
    N.check(code, "sparse_mla_decode")
    return out, lse
