"""Symmetric heap: one IPC-shared slab per rank, with every pool carved out of it.

``SymmetricHeap(group, rank, world, bytes)`` allocates a slab with plain
``cudaMalloc`` (outside the framework allocator, so the CUDA IPC handle covers
exactly this slab), exchanges handles over the CPU (gloo) group and maps every
peer's slab.  ``alloc(name, shape, dtype)`` bump-allocates the same offsets on
every rank, so ``peer_ptr(rank, tensor)`` is plain pointer arithmetic.

All ranks must sit on one host (peer mappings are NVLink/PCIe P2P).  With one
rank, or on CPU, the heap degrades to ordinary tensors and no IPC happens.

Reference: FlowKVPeerShards (ulacache/transfer/ipc.py:12-76: handle exchange with
all_gather_object, same-host check :35-37, pointer-table tensor) and the
flags/step publication of ulacache/transfer/ipc.py:81-101.
"""
from __future__ import annotations

import ctypes as C
import socket

_ALIGN = 1024


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view slab memory."""

    def __init__(self, ptr, nbytes, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}
        self._owner = owner


class SymmetricHeap:
    def __init__(self, *, cpu_group=None, rank: int = 0, world_size: int = 1, nbytes: int, device):
        import torch

        self.rank, self.world, self.device = rank, world_size, torch.device(device)
        self.nbytes = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
        self.cpu_group = cpu_group
        self._cursor = 0
        self._allocs = {}
        self._native = None
        self.base = 0
        self.peer_bases = [0] * world_size
        self.peer_devices = [0] * world_size
        self._opened = []
        self._flag_epoch = 0
        if self.device.type != "cuda":
            self._host = torch.zeros(self.nbytes, dtype=torch.uint8)
            self.base = self._host.data_ptr()
            self.peer_bases[rank] = self.base
            self._view = self._host
            return
        from ..ops import _native as N

        self._native = N
        torch.cuda.set_device(self.device)
        out = C.c_void_p()
        N.check(N.cuda().ulc_slab_alloc(C.byref(out), C.c_ulonglong(self.nbytes)), "slab_alloc")
        self.base = out.value
        self._view = torch.as_tensor(_CudaArray(self.base, self.nbytes, self), device=self.device)
        self.peer_bases[rank] = self.base
        if world_size > 1:
            self._exchange_handles()
        # flags page + pointer tables live at the front of every slab
        self.flags = self.alloc("__flags__", (64,), torch.int32)
        self.status = N.new_status(self.device)
        self._flag_ptrs = torch.tensor([self.peer_ptr(r, self.flags) for r in range(world_size)],
                                       dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------ set-up --
    def _exchange_handles(self):
        import torch.distributed as dist

        N = self._native
        handle = (C.c_ubyte * 64)()
        offset = C.c_ulonglong()
        N.check(N.cuda().ulc_ipc_get_handle(C.c_void_p(self.base), handle, C.byref(offset)), "ipc_get_handle")
        mine = (socket.gethostname(), bytes(handle), int(offset.value))
        mine = mine + (int(self.device.index or 0),)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, mine, group=self.cpu_group)
        if len({g[0] for g in gathered}) != 1:
            raise RuntimeError("All ranks of a symmetric heap must run on one host")
        self.peer_devices = [g[3] for g in gathered]          # CUDA device ordinal of every rank
        for r, (_, h, off, _dev) in enumerate(gathered):
            if r == self.rank:
                continue
            out = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            N.check(N.cuda().ulc_ipc_open_handle(buf, C.byref(out)), f"ipc_open_handle(rank {r})")
            self._opened.append(out.value)                    # mappings this heap must close itself
            self.peer_bases[r] = out.value + off
        dist.barrier(group=self.cpu_group)

    # --------------------------------------------------------------- allocation --
    def alloc(self, name: str, shape, dtype):
        """Same call sequence on every rank yields the same offsets everywhere."""
        import torch

        if name in self._allocs:
            raise KeyError(f"{name} already allocated on this heap")
        itemsize = torch.empty((), dtype=dtype).element_size()
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * itemsize
        start = (self._cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        if start + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted allocating {name} ({nbytes} bytes)")
        self._cursor = start + nbytes
        t = self._view[start:start + nbytes].view(dtype).view(*shape)
        self._allocs[name] = (start, nbytes)
        return t

    def offset_of(self, tensor) -> int:
        return tensor.data_ptr() - self.base

    def peer_ptr(self, rank: int, tensor) -> int:
        return self.peer_bases[rank] + self.offset_of(tensor)

    def peer_ptrs(self, tensor):
        return [self.peer_ptr(r, tensor) for r in range(self.world)]

    @property
    def used_bytes(self) -> int:
        return self._cursor

    # ------------------------------------------------------------------ barrier --
    def device_barrier(self, *, limit_cycles: int = 0):
        """Cross-rank barrier on the current stream, made of system-scope flag stores and
        bounded waits (no NCCL).  A timeout is written to ``self.status``."""
        if self.world == 1 or self._native is None:
            return
        N = self._native
        N.check(N.cuda().ulc_step_barrier(N.ptr(self._flag_ptrs), C.c_int(self.rank), C.c_int(self.world),
                                          C.c_longlong(limit_cycles), N.ptr(self.status), N.stream()),
                "step_barrier")

    def native_atomics_supported(self) -> bool:
        if self._native is None or self.world == 1:
            return True
        N = self._native
        ok = True
        for peer in range(self.world):
            if peer == self.rank:
                continue
            flag = C.c_int()
            # ranks are not device ordinals: ask about the device the peer rank actually runs on
            N.check(N.cuda().ulc_p2p_native_atomics(C.c_int(self.device.index or 0),
                                                    C.c_int(self.peer_devices[peer]), C.byref(flag)),
                    "p2p_native_atomics")
            ok = ok and bool(flag.value)
        return ok

    def close(self, collective: bool = True):
        """Unmap the peers' slabs and free this rank's.  ``collective=False`` skips the barrier with the peers:
        for a rank whose peers are known to be gone, or that has agreed on the order of frees by other means."""
        import torch

        if self._native is not None and self.base:
            if collective and self.world > 1 and self.cpu_group is not None:
                import torch.distributed as dist

                torch.cuda.synchronize()
                dist.barrier(group=self.cpu_group)   # nobody frees while a peer may still read
            for base in self._opened:                         # only this heap's mappings: others stay usable
                self._native.cuda().ulc_ipc_close_handle(C.c_void_p(base))
            self._opened = []
            self._view = None
            self._native.cuda().ulc_slab_free(C.c_void_p(self.base))
            self.base = 0
