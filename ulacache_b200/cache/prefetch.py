"""Follower-layer prefetch: the anchor layer of a residency domain moves its records inside the
step; the same plan's records of the follower layers are copied on a side stream while the anchor
computes, and each follower waits on an event just before it reads.

``completion = "layer"`` records one event per follower layer (a follower can start as soon as its
own bytes have arrived), ``"group"`` one event for the whole domain.

Reference: ulacache/cache/prefetch.py:1-219, cache_config.py:7 (PrefetchPolicy).
"""
from __future__ import annotations

from typing import Callable, Dict, Sequence


class FollowerPrefetcher:
    def __init__(self, policy, backend: str, *, side_stream=None):
        self.policy = policy
        self.completion = policy.resolved_completion(backend)
        self.side = side_stream
        self._events: Dict[int, object] = {}
        self.launched = 0

    def launch(self, followers: Sequence[int], copy_layer: Callable[[int], None]):
        """Run ``copy_layer(l)`` for every follower, on the side stream when there is one."""
        if not self.policy or not followers:
            for l in followers:
                copy_layer(l)
            return
        import torch

        cuda = self.side is not None and torch.cuda.is_available()
        if cuda:
            self.side.wait_stream(torch.cuda.current_stream())
        ctx = torch.cuda.stream(self.side) if cuda else _Null()
        with ctx:
            group_event = None
            for l in followers:
                copy_layer(l)
                self.launched += 1
                if cuda and self.completion == "layer":
                    ev = torch.cuda.Event()
                    ev.record(self.side)
                    self._events[l] = ev
            if cuda and self.completion == "group":
                group_event = torch.cuda.Event()
                group_event.record(self.side)
                for l in followers:
                    self._events[l] = group_event

    def wait(self, layer: int):
        """Make the current stream wait for ``layer``'s prefetched bytes (no-op if none pending)."""
        ev = self._events.pop(layer, None)
        if ev is not None:
            import torch

            torch.cuda.current_stream().wait_event(ev)

    def pending(self) -> int:
        return len(self._events)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


# ----------------------------------------------------------------------------------------------
# Lifecycle of a forward over shared-selection groups.
#
# The anchor layer of a group produces the selection; it is planned ONCE (residency decision,
# resolve) and its records are pulled; the follower layers reuse the plan and only need their own
# bytes.  With prefetch the plan and the anchor's pull run on a side stream from the moment the
# selection exists, and the followers' pulls are queued when the anchor's attention has been
# launched; each consumer joins exactly the event it needs (per layer or per group).  The class
# keeps the forward honest: one plan per anchor, followers scheduled by their anchor, a join before
# a follower prepares, every layer consumed before the forward ends, and an abort that drains the
# side stream before anything is released.
#
# Reference: ulacache/cache/prefetch.py:4-219 (SharedIndexLifecycle.begin_forward /
# join_idle_prefetch / before_layer_prepare / on_index_ready / before_history_consume /
# after_attention / finish_forward / abort_forward).
# ----------------------------------------------------------------------------------------------
class SharedSelectionLifecycle:
    def __init__(self, groups, *, plan_selection: Callable, pull_history: Callable, publish_step: Callable = None,
                 prefetch=False, backend: str = "native_paged", runtime=None):
        """``groups``: :class:`~ulacache_b200.cache.layers.LayerGroupPlan`.  ``plan_selection(layer, selection)``
        plans the anchor's selection; ``pull_history(layer, is_anchor)`` moves the layer's records;
        ``publish_step()`` tells the peers that this rank's readers have retired.  ``prefetch``: bool or
        :class:`~ulacache_b200.cache_config.PrefetchPolicy`.  ``runtime``: stream runtime (CUDA or host)."""
        from ..cache_config import PrefetchPolicy

        policy = PrefetchPolicy(enabled=prefetch) if type(prefetch) is bool else prefetch
        if not isinstance(policy, PrefetchPolicy):
            raise TypeError("prefetch is a bool or a PrefetchPolicy")
        self.groups, self.plan_selection, self.pull_history, self.publish_step = groups, plan_selection, pull_history, publish_step
        self.prefetch = policy.enabled
        self.completion = policy.resolved_completion(backend)
        self._planned = None
        self._consumed, self._keepalive = set(), {}
        self._scheduled, self._joined = set(), set()
        self.plans = self.pulls = 0
        if self.prefetch:
            if runtime is None:
                from ..transfer.prefill_pipeline import HostStreamRuntime

                runtime = HostStreamRuntime()
            self.runtime = runtime
            self._stream = runtime.make_stream()
            self._anchor_ready = tuple(runtime.make_event() for _ in range(groups.group_count))
            self._followers_ready = tuple(runtime.make_event() if f and self.completion == "group" else None
                                          for f in groups.followers)
            self._layer_ready = tuple(runtime.make_event() if self.completion == "layer" and l not in groups.anchors else None
                                      for l in range(groups.layer_count))

    @property
    def in_forward(self) -> bool:
        return self._planned is not None

    def begin_forward(self):
        if self.in_forward:
            raise RuntimeError("the previous shared-selection forward has not finished")
        self._planned = set()
        self._consumed.clear()
        self._scheduled.clear()
        self._joined.clear()

    def join_idle_prefetch(self):
        """Order a mutation outside forwards (release, clear, restore) after every queued pull."""
        if self.in_forward:
            raise RuntimeError("history storage cannot change during a forward")
        if self.prefetch:
            self.runtime.wait_stream(self.runtime.current_stream(), self._stream)

    def before_layer_prepare(self, layer: int):
        """A follower joins its completion boundary before its queries are prepared."""
        if not self.prefetch:
            return
        g = self.groups.group(layer)
        followers = self.groups.followers[g]
        if layer in followers and (self.completion == "layer" or layer == followers[0]):
            key = layer if self.completion == "layer" else ("group", g)
            if key not in self._scheduled:
                raise RuntimeError("a follower's history must be scheduled by its anchor")
            ev = self._layer_ready[layer] if self.completion == "layer" else self._followers_ready[g]
            self.runtime.wait_event(self.runtime.current_stream(), ev)
            self._joined.add(key)

    def _plan(self, layer, selection):
        g = self.groups.group(layer)
        if self.groups.anchors[g] != layer or g in self._planned:
            raise RuntimeError("exactly one selection plans each anchor")
        self.plan_selection(layer, selection)
        self._keepalive[g] = selection            # the plan's source stays alive while pulls may read it
        self._planned.add(g)
        self.plans += 1

    def _pull(self, layer):
        g = self.groups.group(layer)
        self.pull_history(layer, layer == self.groups.anchors[g])
        self.pulls += 1

    def on_selection_ready(self, layer: int, selection):
        if not self.in_forward:
            raise RuntimeError("begin_forward() first")
        if not self.prefetch:
            self._plan(layer, selection)
            return
        rt = self.runtime
        rt.wait_stream(self._stream, rt.current_stream())
        with rt.stream_scope(self._stream):
            self._plan(layer, selection)
            self._pull(layer)
            rt.record_event(self._anchor_ready[self.groups.group(layer)], self._stream)

    def before_history_consume(self, layer: int):
        g = self.groups.group(layer)
        if self._planned is None or g not in self._planned:
            raise RuntimeError("the layer's history has no selection plan")
        if not self.prefetch:
            self._pull(layer)
            return
        if layer == self.groups.anchors[g]:
            # the layer's writer reads what the plan decided: join before the writer, not after it
            self.runtime.wait_event(self.runtime.current_stream(), self._anchor_ready[g])
        elif (layer if self.completion == "layer" else ("group", g)) not in self._joined:
            raise RuntimeError("a follower's history must be joined before its queries are prepared")

    def after_attention(self, layer: int):
        self._consumed.add(layer)
        g = self.groups.group(layer)
        followers = self.groups.followers[g]
        if self.prefetch and layer == self.groups.anchors[g] and followers:
            rt = self.runtime
            rt.wait_stream(self._stream, rt.current_stream())
            with rt.stream_scope(self._stream):
                for f in followers:
                    self._pull(f)
                    if self.completion == "layer":
                        rt.record_event(self._layer_ready[f], self._stream)
                        self._scheduled.add(f)
                if self.completion == "group":
                    rt.record_event(self._followers_ready[g], self._stream)
                    self._scheduled.add(("group", g))

    def finish_forward(self):
        if self._consumed != set(range(self.groups.layer_count)):
            missing = sorted(set(range(self.groups.layer_count)) - self._consumed)
            raise RuntimeError(f"the forward ended with unconsumed layers {missing}")
        if self.prefetch:
            self.runtime.wait_stream(self.runtime.current_stream(), self._stream)
        if self.publish_step is not None:
            self.publish_step()
        self._planned = None
        self._keepalive.clear()

    def abort_forward(self):
        """Drain the queued pulls before the tensors of a partial forward are released."""
        try:
            if self.prefetch:
                self.runtime.synchronize(self._stream)
        finally:
            self._planned = None
            self._consumed.clear()
            self._keepalive.clear()
            self._scheduled.clear()
            self._joined.clear()
