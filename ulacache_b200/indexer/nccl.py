"""Library all-gather of Index score slices with an owner object that fixes its bounds before graph capture.

The fused candidate exchange is the product path; this owner is the fallback transport
(``index_score_transport: "nccl"``) and the baseline it is measured against.  It owns ONE gather
workspace sized from the serving bounds, so a captured decode graph never allocates: every call gathers
into a prefix of that workspace and returns a view of it.  It refuses what a capture could not replay (a
different bound, a foreign output buffer, a misaligned or non-contiguous slice, construction or closing
while a stream is capturing), runs the collective once at construction so the communicator exists before
the first capture, and closes behind a barrier so that no peer still gathers into freed memory.

Score layout: a context of ``max_page_width`` pages is striped over the ranks page by page, so a rank
scores ``ceil(max_page_width / world)`` pages of 64 tokens; a slice is fp32 ``[queries, local_columns]``
and the gathered result ``[world, queries, local_columns]`` in rank order.

Works on CPU tensors with a gloo group (the two-rank tests) and on CUDA tensors with NCCL.

Reference: ulacache/indexer/nccl.py:6-110 (``NCCLIndexOwner``: bounds, workspace, ``validate_bounds``,
``graph_capture``, ``all_gather_into_tensor``, ``close``).
"""
from __future__ import annotations

from contextlib import contextmanager

from ..flashag import IndexTransport

PAGE_TOKENS = 64


def local_score_columns(max_page_width: int, world: int) -> int:
    """Score columns of one rank for contexts of up to ``max_page_width`` pages striped over ``world`` ranks."""
    return (max_page_width + world - 1) // world * PAGE_TOKENS


class CollectiveIndexOwner(IndexTransport):
    def __init__(self, group, *, rank: int, world: int, max_queries: int, max_page_width: int, device,
                 cpu_group=None, warm_up: bool = True):
        import torch

        for name, n in (("max_queries", max_queries), ("max_page_width", max_page_width)):
            if not isinstance(n, int) or isinstance(n, bool) or n < 1:
                raise ValueError(f"{name} must be a positive integer")
        if world < 1 or not 0 <= rank < world:
            raise ValueError("rank outside the group")
        self.device = torch.device(device)
        if self.device.type == "cuda":
            if self.device.index is None:
                self.device = torch.device("cuda", torch.cuda.current_device())
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("construct the Index owner before graph capture")
        self.group, self.cpu_group = group, cpu_group if cpu_group is not None else group
        self.rank, self.world = rank, world
        self.max_queries, self.max_page_width = max_queries, max_page_width
        self.local_columns = local_score_columns(max_page_width, world)
        self.maximum_gather_bytes = world * max_queries * self.local_columns * 4
        self.gathered_workspace = torch.empty(self.maximum_gather_bytes // 4, dtype=torch.float32, device=self.device)
        self.calls = 0
        self._capturing = False
        self._closed = False
        if warm_up and world > 1:
            # the library creates its communicator lazily: do that outside any capture
            self.all_gather_into_tensor(torch.zeros((1, 4), dtype=torch.float32, device=self.device))
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.calls = 0

    # ------------------------------------------------------------------ bounds --
    def validate_bounds(self, max_queries: int, max_page_width: int):
        """A second user of the same owner (another layer group, another captured batch size) must have been
        built for exactly these bounds, or its graph would index past the workspace."""
        if self._closed:
            raise RuntimeError("Index owner is closed")
        if (max_queries, max_page_width) != (self.max_queries, self.max_page_width):
            raise ValueError(f"shared Index owner was built for {(self.max_queries, self.max_page_width)}, "
                             f"not {(max_queries, max_page_width)}")

    @contextmanager
    def graph_capture(self):
        """Wrap a CUDA graph capture: inside it only workspace-backed gathers are accepted."""
        if self._closed:
            raise RuntimeError("Index owner is closed")
        self._capturing = True
        try:
            yield self
        finally:
            self._capturing = False

    # ------------------------------------------------------------------ gather --
    def _check(self, local):
        import torch

        if self._closed:
            raise RuntimeError("Index owner is closed")
        if local.ndim != 2 or local.dtype != torch.float32 or local.device != self.device:
            raise ValueError("a score slice is an fp32 [queries, columns] tensor on the owner's device")
        if not local.is_contiguous() or local.numel() == 0:
            raise ValueError("a score slice must be contiguous and non-empty")
        if local.data_ptr() % 16 or (local.numel() * 4) % 16:
            raise ValueError("a score slice must start on and span a multiple of 16 bytes")
        if local.numel() * 4 * self.world > self.maximum_gather_bytes:
            raise ValueError(f"{tuple(local.shape)} x {self.world} ranks exceeds the owner's bounds "
                             f"({self.max_queries} queries x {self.local_columns} columns)")

    def all_gather_into_tensor(self, local, output=None):
        """Gather ``local`` fp32 [queries, columns] from every rank into the workspace; returns the
        [world * queries, columns] view (rank-major).  ``output``, when given, must BE that view."""
        import torch
        import torch.distributed as dist

        self._check(local)
        q, cols = local.shape
        view = self.gathered_workspace[: self.world * q * cols].view(self.world * q, cols)
        if output is not None and (output.data_ptr() != view.data_ptr() or tuple(output.shape) != tuple(view.shape)
                                   or not output.is_contiguous()):
            raise ValueError("the output of an Index gather is the owner's workspace prefix")
        if self.world == 1:
            view.copy_(local)
        elif self.device.type == "cuda":
            dist.all_gather_into_tensor(view, local, group=self.group)
        else:
            dist.all_gather(list(view.view(self.world, q, cols).unbind(0)), local, group=self.group)
        self.calls += 1
        return view

    def all_gather_scores(self, local):
        """Transport interface: fp32 [rows, cols] -> fp32 [world, rows, cols] (a view of the workspace, valid
        until the next gather)."""
        local = local if local.is_contiguous() else local.contiguous()
        if self._capturing and local.data_ptr() % 16:
            raise ValueError("inside a capture the slice must already be aligned")
        rows, cols = local.shape
        return self.all_gather_into_tensor(local).view(self.world, rows, cols)

    # ------------------------------------------------------------------- close --
    def close(self):
        import torch
        import torch.distributed as dist

        if self._closed:
            return
        if self.device.type == "cuda":
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("cannot close an Index owner during graph capture")
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.cpu_group)       # nobody frees while a peer may still gather
        self.gathered_workspace = None
        self._closed = True


# the stateless form (allocates its output per call; eager experiments)
from ..flashag import CollectiveScoreAllGather as NcclScoreAllGather  # noqa: E402,F401
