"""Passive capture of the rows a tensor-parallel rank found missing locally, frame by frame, in a
chunked device buffer that the host drains at chunk boundaries.

A frame is one forward step; ``control`` holds (enabled, frame number, valid query rows, error bits)
on the device so that recording can be switched and advanced without re-capturing a CUDA graph.

Reference: ulacache/telemetry/tp_sparse_trace.py:4-63 (GpuTpMissTrace),
ulacache/csrc/telemetry/tp_sparse_trace.cuh:10-37.
"""
from __future__ import annotations

import ctypes as C


class GpuTpMissTrace:
    def __init__(self, *, groups: int, query_rows: int, topk: int, frames: int, chunk_frames: int, device,
                 max_gpu_bytes: int = 3_000_000_000):
        import torch

        size = chunk_frames * groups * query_rows * (topk + 1) * 4 + chunk_frames * groups * 4
        if size > max_gpu_bytes:
            raise ValueError("the miss trace exceeds its diagnostic allowance")
        self.groups, self.bound, self.topk, self.frames, self.chunk_frames = groups, query_rows, topk, frames, chunk_frames
        slots = chunk_frames * groups
        i32 = dict(dtype=torch.int32, device=device)
        self.rows = torch.full((slots, query_rows, topk), -1, **i32)
        self.counts = torch.full((slots, query_rows), -1, **i32)
        self.source_rows = torch.zeros(slots, **i32)
        self.control = torch.zeros(4, dtype=torch.int64, device=device)

    @property
    def gpu_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.rows, self.counts, self.source_rows))

    def begin_frame(self, frame: int, valid_query_rows: int, enabled: bool = True):
        import torch

        self.control[:3] = torch.tensor([int(enabled), frame, valid_query_rows], dtype=torch.int64)

    def observe(self, group: int, rows, counts):
        """``rows`` int32 [source rows, topk] local-miss ids per query (first ``counts[q]`` valid)."""
        if not 0 <= group < self.groups:
            raise ValueError("invalid management group")
        if rows.is_cuda:
            from ..ops import _native as N

            N.check(N.cuda().ulc_tp_miss_trace(
                N.ptr(rows), C.c_longlong(rows.stride(0)), N.ptr(counts), C.c_int(rows.shape[0]), N.ptr(self.control),
                N.ptr(self.rows), N.ptr(self.counts), N.ptr(self.source_rows), C.c_int(group), C.c_int(self.frames),
                C.c_int(self.chunk_frames), C.c_int(self.groups), C.c_int(self.bound), C.c_int(self.topk), N.stream()),
                "tp_miss_trace")
            return
        enabled, frame, valid, _ = (int(v) for v in self.control.tolist())
        if not enabled or not 0 <= frame < self.frames:
            return
        if valid < 0 or valid > rows.shape[0] or valid > self.bound:
            self.control[3] |= 1
            return
        slot = (frame % self.chunk_frames) * self.groups + group
        self.rows[slot].fill_(-1)
        self.counts[slot].fill_(-1)
        for q in range(valid):
            n = int(counts[q])
            if n < 0 or n > self.topk:
                self.control[3] |= 2
                n = max(0, min(n, self.topk))
            self.rows[slot, q, :n] = rows[q, :n]
            self.counts[slot, q] = int(counts[q])
        self.source_rows[slot] = rows.shape[0]

    def snapshot_chunk(self) -> dict:
        """Call at a synchronising chunk boundary."""
        if int(self.control[3]):
            raise RuntimeError(f"the miss trace recorded error bits {int(self.control[3])}")
        return dict(local_miss_rows=self.rows.cpu(), local_miss_counts=self.counts.cpu(),
                    source_bucket_rows=self.source_rows.cpu())
