"""Executor of boundary transactions: moves whole pages between the device pool and the pinned
host pool, wave by wave, on a boundary stream, then publishes the new page map.

Offloads of a wave run before its onloads (the onloads reuse the device pages the offloads free).
Copies are pinned ``cudaMemcpyAsync`` calls issued one per page and layer range (``Tensor.copy_``
with ``non_blocking``) on a side stream; on CPU tensors they are plain copies.

Reference: ulacache/transfer/page_exchange.py:53-145.
"""
from __future__ import annotations


class PageExchangeExecutor:
    def __init__(self, storage, *, stream=None, extra_storages=()):
        """``storage``: the record pages; ``extra_storages``: further page pools that move with the same
        page numbers (the Index pages of the anchor layers).  Each has ``device_pool`` / ``host_pool``
        ``[layers, pages, page_bytes]``."""
        self.storage = storage
        self.storages = (storage,) + tuple(extra_storages)
        self.stream = stream
        self.bytes_d2h = 0
        self.bytes_h2d = 0

    def _run_wave(self, wave):
        for st in self.storages:
            per_page = st.page_bytes * st.layers
            for _, dp, hp in wave.offloads:
                st.host_pool[:, hp].copy_(st.device_pool[:, dp], non_blocking=True)
                self.bytes_d2h += per_page
            for _, hp, dp in wave.onloads:
                st.device_pool[:, dp].copy_(st.host_pool[:, hp], non_blocking=True)
                self.bytes_h2d += per_page

    def move(self, txn):
        """Run every wave of ``txn`` (bytes only; nothing is committed or published).  On GPUs the copies run
        on the boundary stream and the current stream waits for them."""
        import torch

        use_stream = self.stream is not None and self.storage.device_pool.is_cuda
        if use_stream:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                for wave in txn.waves:
                    self._run_wave(wave)
            torch.cuda.current_stream().wait_stream(self.stream)
        else:
            for wave in txn.waves:
                self._run_wave(wave)
        return txn.moved_pages

    def execute(self, pool, txn, *, page_map_out=None):
        """Run every wave of ``txn``, commit it, and refresh ``page_map_out`` (device int32) if given."""
        moved = self.move(txn)
        pool.commit(txn)
        if page_map_out is not None:
            page_map_out.copy_(pool.page_map(), non_blocking=True)
        return moved
