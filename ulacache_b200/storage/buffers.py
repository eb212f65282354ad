"""Physical storage of record planes: HBM planes plus a pinned host pool.

The HBM plane of one rank is ``uint8[layers, hbm_slots, record_bytes]``; the
host pool has the same shape with ``host_slots`` rows and lives in pinned memory,
which CUDA maps into the device address space at the same address (unified
addressing), so exchange kernels read and write it directly over PCIe.

Reference: ulacache/storage/buffers.py (RecordPlaneStorage :8,
validate_host_allocation_headroom :338, PinnedHostRecordPool :383).
"""
from __future__ import annotations

from dataclasses import dataclass

from .layout import KeyValueRecordPlane

HOST_HEADROOM_BYTES = 8 << 30      # leave this much MemAvailable after pinning
HOST_HEADROOM_FRACTION = 0.05


def read_meminfo(path="/proc/meminfo") -> dict:
    out = {}
    try:
        with open(path) as f:
            for line in f:
                k, _, rest = line.partition(":")
                parts = rest.split()
                if parts:
                    out[k.strip()] = int(parts[0]) * (1024 if len(parts) > 1 and parts[1] == "kB" else 1)
    except OSError:
        pass
    return out


def validate_host_allocation_headroom(requested_bytes: int, *, meminfo=None,
                                      headroom_bytes: int = HOST_HEADROOM_BYTES,
                                      headroom_fraction: float = HOST_HEADROOM_FRACTION) -> int:
    """Refuse to pin more host memory than the machine can spare.  Returns the bytes
    that would remain available.  Pinned pages cannot be swapped, so an oversized
    pool takes the node down rather than failing an allocation."""
    info = read_meminfo() if meminfo is None else meminfo
    available = info.get("MemAvailable")
    if available is None:
        return -1      # unknown platform: let the allocation itself decide
    total = info.get("MemTotal", available)
    need_left = max(min(headroom_bytes, total // 4), int(total * headroom_fraction))
    left = available - requested_bytes
    if left < need_left:
        raise MemoryError(
            f"Pinning {requested_bytes} bytes would leave {left} bytes available; "
            f"{need_left} must remain (MemAvailable {available})")
    return left


class PinnedHostRecordPool:
    """``uint8[layers, slots, record_bytes]`` in page-locked host memory."""

    def __init__(self, *, layers: int, slots: int, row_bytes: int, device=None, pin: bool = True):
        import torch

        self.layers, self.slots, self.row_bytes = layers, slots, row_bytes
        self.nbytes = layers * slots * row_bytes
        use_pin = pin and torch.cuda.is_available()
        if use_pin:
            validate_host_allocation_headroom(self.nbytes)
        self.storage = torch.zeros((layers, max(slots, 1), row_bytes), dtype=torch.uint8, pin_memory=use_pin)
        self.pinned = use_pin
        self.ptrs = [self.storage[l].data_ptr() for l in range(layers)]

    @property
    def base_ptr(self) -> int:
        return self.storage.data_ptr()

    @property
    def layer_stride(self) -> int:
        return self.storage.stride(0)

    def close(self):
        self.storage = None
        self.ptrs = []


def default_host_pool_factory(*, layers, slots, row_bytes, device=None):
    return PinnedHostRecordPool(layers=layers, slots=slots, row_bytes=row_bytes, device=device)


GUARD_ROWS = 4
GUARD_BYTE = 0xA5


def canaries_enabled(environ=None) -> bool:
    """``ULC_CANARY=1``: a debug build of the record storage.  Every layer's device plane and host plane gets
    ``GUARD_ROWS`` guard records before its first slot and after its last, filled with ``GUARD_BYTE``; ``check``
    on the cache verifies them, so a kernel that writes outside its plane is caught at the next check instead of
    corrupting a neighbouring layer's records."""
    import os

    return (environ if environ is not None else os.environ).get("ULC_CANARY", "0") == "1"


@dataclass
class PlaneGeometry:
    layers: int
    hbm_slots: int
    host_slots: int
    record_bytes: int


class RecordPlaneStorage:
    """One plane's HBM rows and (optionally) host rows for every layer that owns storage."""

    def __init__(self, plane: KeyValueRecordPlane, *, layers: int, hbm_slots: int, host_slots: int,
                 device, host_pool_factory=default_host_pool_factory):
        import torch

        self.plane = plane
        self.geometry = PlaneGeometry(layers, hbm_slots, host_slots, plane.bytes_per_record)
        self.device = torch.device(device)
        self.guard = GUARD_ROWS if canaries_enabled() else 0
        g = self.guard
        self._device_block = torch.zeros((layers, hbm_slots + 2 * g, plane.bytes_per_record), dtype=torch.uint8,
                                         device=self.device)
        self.gpu = self._device_block[:, g:g + hbm_slots] if g else self._device_block
        self.host_pool = None
        if host_slots > 0:
            if self.device.type == "cuda":
                self.host_pool = host_pool_factory(layers=layers, slots=host_slots + 2 * g,
                                                   row_bytes=plane.bytes_per_record, device=self.device)
            else:
                self.host_pool = PinnedHostRecordPool(layers=layers, slots=host_slots + 2 * g,
                                                      row_bytes=plane.bytes_per_record, pin=False)
        if g:
            for block in (self._device_block, None if self.host_pool is None else self.host_pool.storage):
                if block is not None:
                    block[:, :g] = GUARD_BYTE
                    block[:, block.shape[1] - g:] = GUARD_BYTE

    @property
    def host(self):
        if self.host_pool is None:
            return None
        g = self.guard
        return self.host_pool.storage[:, g:g + self.geometry.host_slots] if g else self.host_pool.storage

    def check_canaries(self):
        """Raise when a guard record of any layer has been overwritten (no-op without ``ULC_CANARY=1``)."""
        g = self.guard
        if not g:
            return
        for tier, block in (("device", self._device_block),
                            ("host", None if self.host_pool is None else self.host_pool.storage)):
            if block is None:
                continue
            for side, rows in (("before", block[:, :g]), ("after", block[:, block.shape[1] - g:])):
                bad = (rows != GUARD_BYTE).reshape(rows.shape[0], -1).any(dim=1)
                if bool(bad.any()):
                    layers = bad.nonzero().flatten().tolist()
                    raise RuntimeError(f"plane {self.plane.name!r}: guard records {side} the {tier} slots of storage "
                                       f"layer(s) {layers} were overwritten")

    def device_bytes(self) -> int:
        return self._device_block.numel()

    def host_bytes(self) -> int:
        return 0 if self.host_pool is None else self.host_pool.nbytes

    def close(self):
        if self.host_pool is not None:
            self.host_pool.close()
        self.host_pool = None
        self.gpu = self._device_block = None
