"""Per-kernel timing of the engine's steps with CUDA events.

The reference wraps each operation of a layer in an event pair and prints time
shares, TFLOP/s and GB/s per operation name (src/profiler/profiler.ts:93-479).
Here the event pairs sit around every kernel launch of the engine's library and
every library matrix product, while CUDA graphs are off; ``framework`` is the
wall time that no kernel accounts for, as in the reference (:197-282).
"""
from __future__ import annotations

import json
import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch

from .csrc import ops


class Profiler:
    def __init__(self, engine=None):
        self.engine = engine
        self.spans: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self._open: Dict[str, torch.cuda.Event] = {}
        self.t0 = time.perf_counter()
        ops.set_profiler(self)

    def begin(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open[name] = ev

    def end(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.spans.append((name, self._open.pop(name), ev))

    def stop(self) -> None:
        ops.set_profiler(None)

    def collect(self) -> Dict[str, Tuple[int, float]]:
        """name -> (calls, total milliseconds)."""
        torch.cuda.synchronize()
        out: Dict[str, List[float]] = defaultdict(lambda: [0, 0.0])
        for name, a, b in self.spans:
            out[name][0] += 1
            out[name][1] += a.elapsed_time(b)
        return {k: (int(v[0]), float(v[1])) for k, v in out.items()}

    def report(self) -> str:
        self.stop()
        wall = (time.perf_counter() - self.t0) * 1e3
        rows = sorted(self.collect().items(), key=lambda kv: -kv[1][1])
        gpu = sum(ms for _, (_, ms) in rows)
        lines = ["", f"{'operation':<28}{'calls':>8}{'ms':>12}{'share':>9}", "-" * 57]
        for name, (n, ms) in rows:
            lines.append(f"{name:<28}{n:>8}{ms:>12.3f}{100 * ms / max(gpu, 1e-9):>8.1f}%")
        lines.append("-" * 57)
        lines.append(f"{'kernels':<28}{'':>8}{gpu:>12.3f}")
        lines.append(f"{'framework (wall - kernels)':<28}{'':>8}{max(wall - gpu, 0):>12.3f}")
        return "\n".join(lines)

    def write_trace(self, path: str) -> None:
        """Kernel spans in the Chrome tracing format (the reference's tracer:
        src/profiler/tracer.ts)."""
        self.stop()
        torch.cuda.synchronize()
        events = []
        if self.spans:
            origin = self.spans[0][1]
            for name, a, b in self.spans:
                events.append({"name": name, "ph": "X", "pid": 0, "tid": 0,
                               "ts": origin.elapsed_time(a) * 1e3,
                               "dur": a.elapsed_time(b) * 1e3})
        with open(path, "w") as f:
            json.dump({"traceEvents": events}, f)
