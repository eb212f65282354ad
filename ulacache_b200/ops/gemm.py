"""Weight-stationary decode GEMM (tcgen05 + TMA) and its reference."""
from __future__ import annotations

import ctypes as C

from . import _native as N


def linear_reference(x, w):
    """fp32 reference: ``x[T,K] @ w[N,K]^T``."""
    return x.float() @ w.float().t()


def linear(x, w, *, splits: int = 0, status=None, out=None, scratch=None):
    """``y[T,N] = x[T,K] @ w[N,K]^T`` in bf16 with fp32 accumulation on the tensor cores.

    ``splits`` > 1 splits K over CTAs (fp32 scratch of ``T*N`` floats, allocated here
    unless given); 0 picks a split that fills the 148 SMs.
    """
    import torch

    if not x.is_cuda:
        return linear_reference(x, w).to(x.dtype)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1]
    assert x.stride(1) == 1 and w.stride(1) == 1
    T, K = x.shape
    Nout = w.shape[0]
    if out is None:
        out = torch.empty((T, Nout), dtype=torch.bfloat16, device=x.device)
    if splits <= 0:
        bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
        tiles = ((Nout + 127) // 128) * ((T + bn - 1) // bn)
        splits = max(1, min(148 // max(tiles, 1), (K // 64) // 4, 16))
    if splits > 1 and scratch is None:
        scratch = torch.empty((T, Nout), dtype=torch.float32, device=x.device)
    code = N.cuda().ulc_gemm_wt_bf16(
        N.ptr(x), N.ptr(w), N.ptr(out), C.c_int(T), C.c_int(Nout), C.c_int(K),
        C.c_int(x.stride(0)), C.c_int(w.stride(0)), C.c_int(splits), N.ptr(scratch),
        N.ptr(status), N.stream())
    N.check(code, "gemm_wt_bf16")
    return out


MANY_ROWS = 512


def many_rows(t: int) -> bool:
    """Row counts from which the per-head products go to the library's batched GEMM (``ULC_PREFILL_GEMM=0``: never)."""
    import os

    return t >= MANY_ROWS and os.environ.get("ULC_PREFILL_GEMM", "1") != "0"


def batched_linear(x, w, out):
    """For every batch index b: ``out[:, b, :] = x[:, b, :] @ w[b]^T`` on the tensor cores.
    ``x`` bf16 [T, batch, K] (any strides with unit inner stride, multiples of 8), ``w`` bf16
    [batch, N, K] contiguous, ``out`` bf16 [T, batch, N] (any strides).  Used for the per-head
    MLA absorb products, where it reads and writes the head-interleaved layouts in place."""
    import torch

    T, Bt, K = x.shape
    N_ = w.shape[1]
    assert x.stride(2) == 1 and out.stride(2) == 1 and w.is_contiguous() and w.shape[0] == Bt and w.shape[2] == K
    if many_rows(T):
        # prefill-sized row counts: a plain batched bf16 GEMM, which the library does at several times the rate of
        # the decode kernel (built for at most a few dozen rows per head); no epilogue is fused here
        dst = out.permute(1, 0, 2)
        if dst.is_contiguous():
            torch.bmm(x.permute(1, 0, 2), w.transpose(1, 2), out=dst)
        else:
            out.copy_(torch.bmm(x.permute(1, 0, 2), w.transpose(1, 2)).permute(1, 0, 2))
        return out
    code = N.cuda().ulc_gemm_wt_bf16_batched(
        N.ptr(x), N.ptr(w), N.ptr(out), C.c_int(T), C.c_int(N_), C.c_int(K), C.c_longlong(x.stride(0)),
        C.c_longlong(K), C.c_longlong(out.stride(0)), C.c_int(Bt), C.c_longlong(x.stride(1)),
        C.c_longlong(N_ * K), C.c_longlong(out.stride(1)), C.c_int(1), C.c_void_p(0), C.c_void_p(0), N.stream())
    N.check(code, "gemm_wt_bf16")
    return out


def batched_linear_quant(x, w, *, status=None):
    """``batched_linear`` whose result leaves the kernel already quantised for the next fp8 GEMM:
    returns (uint8 fp8 [T, batch * N], fp32 scales [T, batch * N / 128]) with one scale per token
    and 128 output features (``N`` a multiple of 128).  On the CPU: the reference product followed
    by the reference quantiser."""
    import torch
    from . import fp8

    T, Bt, K = x.shape
    N_ = w.shape[1]
    assert N_ % 128 == 0 and w.shape[0] == Bt and w.shape[2] == K
    if not x.is_cuda:
        y = torch.einsum("tbk,bnk->tbn", x.float(), w.float()).reshape(T, Bt * N_)
        return fp8.act_quant_reference(y)
    assert x.stride(2) == 1 and w.is_contiguous()
    if many_rows(T):
        y = torch.bmm(x.permute(1, 0, 2), w.transpose(1, 2)).permute(1, 0, 2).reshape(T, Bt * N_)
        return fp8.act_quant(y)
    q = torch.empty((T, Bt * N_), dtype=torch.uint8, device=x.device)
    sc = torch.empty((T, Bt * N_ // 128), dtype=torch.float32, device=x.device)
    code = N.cuda().ulc_gemm_wt_bf16_batched_quant(
        N.ptr(x), N.ptr(w), N.ptr(q), N.ptr(sc), C.c_int(T), C.c_int(N_), C.c_int(K), C.c_longlong(x.stride(0)),
        C.c_longlong(K), C.c_longlong(Bt * N_), C.c_longlong(Bt * N_ // 128), C.c_int(Bt), C.c_longlong(x.stride(1)),
        C.c_longlong(N_ * K), C.c_longlong(N_), N.ptr(status), N.stream())
    N.check(code, "gemm_wt_bf16_quant")
    return q, sc
