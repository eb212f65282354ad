"""Observability of the cache: sampled hit counters, replay byte metrics, selection traces.

Reference: ulacache/telemetry/cache_hits.py:11, replay_metrics.py:4, sparse_trace.py:74,
tp_sparse_trace.py:4, trace_coverage.py:4.
"""
from .cache_hits import CacheHitSampler  # noqa: F401
from .replay_metrics import DeviceReplayProbes, ReplayMetrics  # noqa: F401
from .sparse_trace import GpuSparseTraceRecorder, load_trace  # noqa: F401
from .tp_sparse_trace import GpuTpMissTrace  # noqa: F401
from .trace_coverage import validate_bucket_rotation, validate_fused_begin_rotation, validate_trace_coverage  # noqa: F401
