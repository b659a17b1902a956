"""Device-timed tracing: CUDA-event timers per module and phase, NVTX ranges, JSON-lines output.

The reference has no tracing of its own (its Fast-Tuner parses vendor profiler CSVs).  Here the
framework produces its own records: ``LayerTimer`` hooks modules and writes
``{"module": kind, "name": fqn, "phase": "fwd"|"bwd", "ms": t, "step": n}`` lines that the
Fast-Tuner profile parser consumes; ``nvtx_range`` marks regions for ncu / other tools.
"""
from __future__ import annotations

import contextlib
import json
from typing import Callable, Dict, List, Optional

import torch
from torch import nn


_NVTX = None


@contextlib.contextmanager
def nvtx_range(name: str):
    global _NVTX
    if _NVTX is None:
        _NVTX = torch.cuda.is_available()
    if _NVTX:
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class CudaTimer:
    """Accumulates CUDA-event durations per key; events are resolved lazily (no sync in the hot path)."""

    def __init__(self):
        self.pending: List[tuple] = []
        self.totals: Dict[str, float] = {}
        self.counts: Dict[str, int] = {}
        self.cuda = torch.cuda.is_available()

    @contextlib.contextmanager
    def time(self, key: str):
        if not self.cuda:
            import time
            t0 = time.perf_counter()
            yield
            self._add(key, (time.perf_counter() - t0) * 1e3)
            return
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        yield
        e.record()
        self.pending.append((key, s, e))

    def start(self, key: str):
        if not self.cuda:
            import time
            return (key, time.perf_counter())          # CPU runs (the gloo tests): host clock
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return (key, ev)

    def stop(self, token) -> None:
        key, s = token
        if not self.cuda:
            import time
            self._add(key, (time.perf_counter() - s) * 1e3)
            return
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pending.append((key, s, e))

    def _add(self, key: str, ms: float) -> None:
        self.totals[key] = self.totals.get(key, 0.0) + ms
        self.counts[key] = self.counts.get(key, 0) + 1

    def resolve(self) -> Dict[str, float]:
        if self.pending:
            torch.cuda.synchronize()
            for key, s, e in self.pending:
                self._add(key, s.elapsed_time(e))
            self.pending = []
        return {k: self.totals[k] / self.counts[k] for k in self.totals}


class LayerTimer:
    """Times forward and backward of selected modules.

    ``classify(name, module) -> kind or None`` tags modules (e.g. ``"dense"``, ``"moe"``, ``"head"``).
    """

    def __init__(self, model: nn.Module, classify: Callable[[str, nn.Module], Optional[str]]):
        self.timer = CudaTimer()
        self.records: List[dict] = []
        self.step = 0
        for name, mod in model.named_modules():
            kind = classify(name, mod)
            if kind is None:
                continue
            self._hook(name, kind, mod)

    def _hook(self, name: str, kind: str, mod: nn.Module) -> None:
        state = {}

        def pre(m, args):
            state["f"] = self.timer.start(f"{kind}|{name}|fwd")

        def post(m, args, out):
            self.timer.stop(state.pop("f"))

        def bpre(m, gout):
            state["b"] = self.timer.start(f"{kind}|{name}|bwd")

        def bpost(m, gin, gout):
            if "b" in state:
                self.timer.stop(state.pop("b"))
        mod.register_forward_pre_hook(pre)
        mod.register_forward_hook(post)
        mod.register_full_backward_pre_hook(bpre)
        mod.register_full_backward_hook(bpost)

    def dump(self, path: str) -> None:
        means = self.timer.resolve()
        with open(path, "a") as f:
            for key, ms in means.items():
                kind, name, phase = key.split("|")
                f.write(json.dumps({"module": kind, "name": name, "phase": phase, "ms": ms, "step": self.step}) + "\n")
