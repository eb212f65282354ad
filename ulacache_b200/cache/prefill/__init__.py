"""Prefill paths of the cache: bounded record windows, the selection union that fills them, leases
on window rows, a read-only reader for cached history, and the per-layer double-buffered pipeline.

Reference: ulacache/cache/prefill/buffers.py, window.py, plans.py, reader.py, leases.py and
transfer/prefill_pipeline.py (LayerPrefillPipeline).
"""
from .buffers import (PrefillQueryGroup, PrefillWindow, PrefillWindowPair, RequestPrefillBuffers,  # noqa: F401
                      prepare_query_groups, request_query_ranges)
from .leases import PrefixPageLeases, WindowLeases, prefill_physical_tokens  # noqa: F401
from .plans import (PrefillChunkPlan, PrefillReadPlans, PrefillSequenceBudget, plan_prefill_chunks,  # noqa: F401
                    prefill_request_groups)
from .reader import HistoryReadPlan, PrefillMaterializer, ReadOnlyPrefillReader, prepare_history_read_plan  # noqa: F401
from .window import (PrefillReadPlan, PrefillRecordWindow, SelectionWindowMap, WindowedPrefillReader,  # noqa: F401
                     compact_selection, shared_union)
