"""Tracing helpers: named phases with NVTX ranges and device time, and the ``--profile`` hook.

The reference only profiles ``interactive.py`` (``torch.profiler`` around the last sample,
interactive.py:416-441) and carries an ``Arguments.profile`` flag that no trainer reads
(arguments.py:283-288). Here the flag is honoured by the trainers: ``StepProfiler`` records a
``torch.profiler`` chrome trace of a few training steps after a warm-up, one file per rank.
``PhaseTimer`` is the device-side stopwatch used around phases of a step: CUDA events on the
current stream (no host synchronisation until the numbers are read), an NVTX range of the same
name for external tools, and ``summary`` reduces with MAX over the ranks, which is the figure
that bounds a synchronous step.
"""
from __future__ import annotations

import contextlib
from collections import defaultdict
from pathlib import Path
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class PhaseTimer:
    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._open: List = []
        self._events: Dict[str, List] = defaultdict(list)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        torch.cuda.nvtx.range_push(name)
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        try:
            yield
        finally:
            e1.record()
            torch.cuda.nvtx.range_pop()
            self._events[name].append((e0, e1))

    def totals_ms(self) -> Dict[str, float]:
        """Device milliseconds per phase on this rank (synchronises once)."""
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self._events.items()}

    def summary(self, group=None) -> Dict[str, float]:
        """Per-phase device milliseconds, MAX over the ranks of ``group``."""
        tot = self.totals_ms()
        if not tot or not (dist.is_available() and dist.is_initialized()):
            return tot
        keys = sorted(tot)
        t = torch.tensor([tot[k] for k in keys], dtype=torch.float32,
                         device=torch.device("cuda", torch.cuda.current_device()))
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        return dict(zip(keys, t.tolist()))

    def reset(self) -> None:
        self._events.clear()


class StepProfiler:
    """``torch.profiler`` over steps ``[skip, skip + active)`` of a loop; the chrome trace goes
    to ``<path>_rank_<r>.json`` (``<path>.json`` without a process group). Call ``step()`` once
    per training step; a ``None`` path makes every call a no-op."""

    def __init__(self, path: Optional[Path], skip: int = 1, active: int = 2):
        self.path = Path(path) if path else None
        self.skip, self.active = skip, active
        self._n = 0
        self._prof = None

    def step(self) -> None:
        if self.path is None:
            return
        if self._n == self.skip:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts)
            self._prof.__enter__()
        elif self._n == self.skip + self.active and self._prof is not None:
            self.close()
        self._n += 1

    def close(self) -> Optional[Path]:
        if self._prof is None:
            return None
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self._prof.__exit__(None, None, None)
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else None
        out = Path(f"{self.path}_rank_{rank}.json" if rank is not None else f"{self.path}.json")
        out.parent.mkdir(parents=True, exist_ok=True)
        self._prof.export_chrome_trace(str(out))
        self._prof = None
        self.path = None
        return out
