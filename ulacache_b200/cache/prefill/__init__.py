"""Prefill paths of the cache: bounded record windows, the selection union that fills them, leases
on window rows, a read-only reader for cached history, and the per-layer double-buffered pipeline.

Reference: ulacache/cache/prefill/buffers.py, window.py, plans.py, reader.py, leases.py and
transfer/prefill_pipeline.py (LayerPrefillPipeline).
"""
from .buffers import PrefillWindow, PrefillWindowPair  # noqa: F401
from .leases import WindowLeases  # noqa: F401
from .plans import PrefillChunkPlan, plan_prefill_chunks  # noqa: F401
from .reader import ReadOnlyPrefillReader  # noqa: F401
from .window import (PrefillReadPlan, PrefillRecordWindow, SelectionWindowMap, WindowedPrefillReader,  # noqa: F401
                     compact_selection, shared_union)
