"""Per-layer double-buffered prefill: while attention of layer l reads window A, the union of layer
l + 1 is gathered into window B on a side stream.

    pipe = LayerPrefillPipeline(reader, map, pair, leases)
    pipe.prime(layer0, selection0)
    for l in layers:
        window, rows = pipe.acquire(l)                 # waits for the fill of l
        if l + 1 < L: pipe.prefetch(l + 1, selection_of(l + 1))
        ... attention reads window.data[rows] ...
        pipe.release(l)

Layers of one shared-selection group pass the same selection; the union map is then computed once.

Reference: ulacache/transfer/prefill_pipeline.py:1-330 (LayerPrefillPipeline).
"""
from __future__ import annotations

from contextlib import contextmanager


class LayerPrefillPipeline:
    def __init__(self, reader, window_map, pair, leases=None, *, side_stream=None):
        from ..cache.prefill.leases import WindowLeases

        self.reader, self.map, self.pair = reader, window_map, pair
        self.leases = leases or WindowLeases()
        self.side = side_stream
        self._pending = {}      # layer -> (window, rows, missing)
        self._tokens = {}
        self._last_sel = None   # (selection object id, union result) reuse inside a group

    def _union(self, selection):
        key = id(selection)
        if self._last_sel is not None and self._last_sel[0] == key:
            return self._last_sel[1]
        res = self.map.build(selection)
        self._last_sel = (key, res)
        return res

    def _fill(self, window, layer, selection):
        import torch

        self.leases.check_refill(window)
        ids, count, rows = self._union(selection)
        if window.data.is_cuda and self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                missing = self.reader.fill(window, layer, ids, count)
        else:
            missing = self.reader.fill(window, layer, ids, count)
        self._pending[layer] = (window, rows, missing)

    def prime(self, layer: int, selection):
        self._fill(self.pair.current, layer, selection)

    def prefetch(self, layer: int, selection):
        self._fill(self.pair.next, layer, selection)

    def acquire(self, layer: int):
        import torch

        if layer not in self._pending:
            raise KeyError(f"layer {layer} was not primed or prefetched")
        window, rows, _ = self._pending[layer]
        if window is not self.pair.current:
            self.pair.swap()
        if window.ready is not None:
            torch.cuda.current_stream().wait_event(window.ready)
        self._tokens[layer] = self.leases.acquire(window)
        return window, rows

    def release(self, layer: int):
        window, _, _ = self._pending.pop(layer)
        self.leases.release(window, self._tokens.pop(layer))


# ----------------------------------------------------------------------------------------------
# Full-history layer pipeline with strict event ordering.
#
# Caller order per forward:   begin(plan) -> for each layer in order:
#     prepare(layer)        prefetch of this layer's window (and of the next layer's into the other window)
#     <the layer's writer produces its current records>
#     read(layer)           waits for the gather, installs the current records once, returns the window
#     <attention>
#     after_attention(layer)    or  skip_unused(layer) when the layer never read its window
# -> finish()   (or abort() after an error).
# A window is never overwritten before the layer that owns it has retired; the pipeline refuses
# out-of-order use instead of corrupting a window.  The backend supplies the two callbacks
# (``gather_history`` on the prefetch stream, ``install_current`` on the caller's stream); this
# class owns streams and events only.
#
# Reference: ulacache/transfer/prefill_pipeline.py:21-330 (PrefillSequenceBudget,
# allocate_native_prefill_windows, CudaPrefillRuntime, LayerPrefillPipeline.begin / prepare / read /
# after_attention / skip_unused / finish / abort / memory_inventory).
# ----------------------------------------------------------------------------------------------

DEFAULT_PREFILL_RECORDS = 1 << 20


def allocate_prefill_windows(device, *, capacity_records: int = DEFAULT_PREFILL_RECORDS, record_bytes: int = 656):
    """Exactly two encoded windows (:class:`~ulacache_b200.cache.prefill.buffers.PrefillWindow`), independently
    owned.  Dequantised outputs and other scratch are the backend's own allocations."""
    from ..cache.prefill.buffers import PrefillWindow

    if type(capacity_records) is not int or capacity_records < 1 or type(record_bytes) is not int or record_bytes < 1:
        raise ValueError("window dimensions must be positive integers")
    return tuple(PrefillWindow(capacity_records, record_bytes, device) for _ in range(2))


class CudaStreamRuntime:
    """Streams and events of one CUDA device."""

    def __init__(self, device):
        import torch

        self.torch, self.device = torch, torch.device(device)

    def make_stream(self):
        return self.torch.cuda.Stream(device=self.device)

    def make_event(self):
        return self.torch.cuda.Event()

    def current_stream(self):
        return self.torch.cuda.current_stream(self.device)

    @contextmanager
    def stream_scope(self, stream):
        with self.torch.cuda.stream(stream):
            yield

    def wait_stream(self, destination, source):
        destination.wait_stream(source)

    def wait_event(self, stream, event):
        stream.wait_event(event)

    def record_event(self, event, stream):
        event.record(stream)

    def record_tensor(self, tensor, stream):
        tensor.record_stream(stream)

    def synchronize(self, stream):
        stream.synchronize()

    def is_capturing(self) -> bool:
        return self.torch.cuda.is_current_stream_capturing()


class HostStreamRuntime:
    """The same interface on the host (CPU tensors, tests): everything runs in call order; ``log`` keeps the
    sequence of stream operations so that tests can check the ordering the CUDA runtime would enforce."""

    def __init__(self):
        self.log = []
        self._n = 0

    def _new(self, kind):
        self._n += 1
        return f"{kind}{self._n}"

    def make_stream(self):
        return self._new("stream")

    def make_event(self):
        return self._new("event")

    def current_stream(self):
        return "main"

    @contextmanager
    def stream_scope(self, stream):
        self.log.append(("enter", stream))
        yield
        self.log.append(("leave", stream))

    def wait_stream(self, destination, source):
        self.log.append(("wait_stream", destination, source))

    def wait_event(self, stream, event):
        self.log.append(("wait_event", stream, event))

    def record_event(self, event, stream):
        self.log.append(("record", event, stream))

    def record_tensor(self, tensor, stream):
        pass

    def synchronize(self, stream):
        self.log.append(("sync", stream))

    def is_capturing(self) -> bool:
        return False


class HistoryPrefillPipeline:
    def __init__(self, windows, *, gather_history, install_current, runtime=None):
        windows = tuple(windows)
        if len(windows) != 2 or windows[0] is windows[1]:
            raise ValueError("two independently owned prefill windows are required")
        if windows[0].data.untyped_storage().data_ptr() == windows[1].data.untyped_storage().data_ptr():
            raise ValueError("the two windows must not alias one allocation")
        if windows[0].capacity != windows[1].capacity or windows[0].record_bytes != windows[1].record_bytes:
            raise ValueError("the two windows must have one geometry")
        if not callable(gather_history) or not callable(install_current):
            raise TypeError("both backend callbacks are required")
        self.windows = windows
        self.capacity_records, self.record_bytes = windows[0].capacity, windows[0].record_bytes
        self.gather_history, self.install_current = gather_history, install_current
        if runtime is None:
            runtime = CudaStreamRuntime(windows[0].data.device) if windows[0].data.is_cuda else HostStreamRuntime()
        self.runtime = runtime
        self.stream = runtime.make_stream()
        self.ready = tuple(runtime.make_event() for _ in windows)
        self.retired = tuple(runtime.make_event() for _ in windows)
        self.forwards = 0
        self._reset()

    def _reset(self):
        self.plan = None
        self.keepalive = ()
        self.layer_count = self.record_count = 0
        self.scheduled, self.installed, self.attended = set(), set(), set()
        self.slot_owner = [None, None]
        self.active_layer = None

    # ------------------------------------------------------------------- forward --
    def begin(self, plan, *, layer_count: int, record_count: int, keepalive_tensors=()):
        if self.plan is not None or self.active_layer is not None:
            raise RuntimeError("finish or abort the previous prefill forward first")
        if self.runtime.is_capturing():
            raise RuntimeError("prefill reconstruction runs eagerly")
        if plan is None or type(layer_count) is not int or layer_count < 1:
            raise ValueError("a plan and a positive layer count are required")
        if type(record_count) is not int or not 0 < record_count <= self.capacity_records:
            raise ValueError("the admitted full-history record count exceeds one window")
        self.plan, self.layer_count, self.record_count = plan, layer_count, record_count
        self.keepalive = tuple(keepalive_tensors)

    def _check_layer(self, layer):
        if self.plan is None or type(layer) is not int or not 0 <= layer < self.layer_count:
            raise ValueError("a valid layer of an active prefill forward is required")

    def _prefetch(self, layer):
        if layer in self.scheduled:
            return
        slot = layer % 2
        previous = self.slot_owner[slot]
        if previous is not None and previous not in self.attended:
            raise RuntimeError("a window would be overwritten before its layer's attention retired")
        rt = self.runtime
        rt.wait_stream(self.stream, rt.current_stream())
        with rt.stream_scope(self.stream):
            if previous is not None:
                rt.wait_event(self.stream, self.retired[slot])
            for t in self.keepalive:
                rt.record_tensor(t, self.stream)
            self.gather_history(layer, self.plan, self.windows[slot])
            rt.record_event(self.ready[slot], self.stream)
        self.scheduled.add(layer)
        self.slot_owner[slot] = layer

    def prepare(self, layer: int):
        self._check_layer(layer)
        if self.active_layer is not None and self.active_layer != layer:
            raise RuntimeError("retire the current attention before preparing another layer")
        if layer != len(self.attended):
            raise RuntimeError("prefill layers are consumed in order")
        self.active_layer = layer
        self._prefetch(layer)
        if layer + 1 < self.layer_count:
            self._prefetch(layer + 1)
        return self.windows[layer % 2]

    def read(self, layer: int):
        self._check_layer(layer)
        if self.active_layer != layer or self.slot_owner[layer % 2] != layer:
            raise RuntimeError("prepare the layer before its read")
        if layer not in self.installed:
            self.runtime.wait_event(self.runtime.current_stream(), self.ready[layer % 2])
            self.install_current(layer, self.plan, self.windows[layer % 2])
            self.installed.add(layer)
        return self.windows[layer % 2]

    def after_attention(self, layer: int):
        self._check_layer(layer)
        if self.active_layer != layer or layer not in self.installed or layer in self.attended:
            raise RuntimeError("retire each consumed prefill layer exactly once")
        self.runtime.record_event(self.retired[layer % 2], self.runtime.current_stream())
        self.attended.add(layer)
        self.active_layer = None

    def skip_unused(self, layer: int):
        """Retire a layer that finished without reading its window (e.g. a first chunk with nothing cached).  A
        prefetched but unread window needs no wait on the caller's stream: the prefetch stream orders its old copy
        before any later overwrite, and the retired event keeps the layer's completion as the boundary."""
        self._check_layer(layer)
        if layer != len(self.attended) or self.active_layer not in (None, layer) or layer in self.installed:
            raise RuntimeError("only the next completed and unread layer can be skipped")
        if layer in self.scheduled:
            self.runtime.record_event(self.retired[layer % 2], self.runtime.current_stream())
        self.attended.add(layer)
        self.active_layer = None

    def finish(self):
        if self.plan is None:
            return
        if self.active_layer is not None or len(self.attended) != self.layer_count:
            raise RuntimeError("unconsumed prefill layers need abort(), not finish()")
        self.runtime.wait_stream(self.runtime.current_stream(), self.stream)
        self.forwards += 1
        self._reset()

    def abort(self):
        self.runtime.synchronize(self.stream)
        self._reset()

    def close(self):
        self.abort()

    def memory_inventory(self) -> dict:
        return dict(capacity_records_per_window=self.capacity_records, record_bytes=self.record_bytes, window_count=2,
                    encoded_window_bytes=sum(w.data.untyped_storage().nbytes() for w in self.windows),
                    excludes_dequantised_output_and_backend_scratch=True)
