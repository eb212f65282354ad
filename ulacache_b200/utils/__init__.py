"""Small shared helpers: device timers, environment flags, JSON-line logging."""
from __future__ import annotations

import json
import os
import sys
import time


def env_flag(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    return default if v is None else v.strip().lower() in ("1", "true", "yes", "on")


class CudaTimer:
    """``with CudaTimer() as t: ...`` then ``t.ms`` (CUDA events on the current stream; wall clock on CPU)."""

    def __enter__(self):
        import torch

        self._cuda = torch.cuda.is_available()
        if self._cuda:
            self._a, self._b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self._a.record()
        else:
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        import torch

        if self._cuda:
            self._b.record()
            torch.cuda.synchronize()
            self.ms = self._a.elapsed_time(self._b)
        else:
            self.ms = (time.perf_counter() - self._t0) * 1e3
        return False


def log_json(stream=None, **fields):
    print(json.dumps(fields), file=stream or sys.stderr, flush=True)


def append_result_csv(path: str, row: dict):
    """Append one result row to an experiment's ``results.csv`` (created with a header on first use; a row with
    new keys rewrites the file with the widened header).  Nested values are stored as JSON text.

    Reference: scripts/7_2_throughput/README.md:50-52 (one ``results.csv`` per experiment)."""
    import csv
    import json
    import os

    flat = {k: (json.dumps(v, sort_keys=True) if isinstance(v, (dict, list, tuple)) else v) for k, v in row.items()}
    rows, header = [], []
    if os.path.exists(path):
        with open(path, newline="") as f:
            reader = csv.DictReader(f)
            header = list(reader.fieldnames or [])
            rows = list(reader)
    new = [k for k in flat if k not in header]
    if not rows and not header:
        header = list(flat)
    elif new:
        header = header + new
    if new or not os.path.exists(path):
        with open(path, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=header)
            w.writeheader()
            w.writerows(rows)
            w.writerow(flat)
        return
    with open(path, "a", newline="") as f:
        csv.DictWriter(f, fieldnames=header).writerow(flat)
