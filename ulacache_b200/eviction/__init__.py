"""Replacement policies of the device tier.

The production policy (a 255-bucket recency ring with a cold bucket) lives in the residency
kernels (``ulacache_b200/csrc/residency.cu``, driven by ``cache/residency.py``).  This package holds
what surrounds it: the CPU oracle for every policy (``oracle``), the ablation policies that replay
the same selection traces on the GPU (``policies``), and launch sizing (``launch_config``).

Reference: ulacache/eviction/lru.py, linked_list_lru.py, hisparse_union.py, trace_hits.py,
launch_config.py.
"""
from .launch_config import LaunchConfig, victim_launch_config  # noqa: F401
from .oracle import POLICY_KINDS, PolicyOracle, replay_trace  # noqa: F401
from .policies import (ExactLruPolicy, HotBufferPolicy, LinkedListLruPolicy, ParallelPresenceRing,  # noqa: F401
                       ParallelPresenceRingPolicy, PresenceRingPolicy, trace_hits)
