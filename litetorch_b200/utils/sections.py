"""Named sections of a step timed with CUDA events (a light substitute for a timeline profiler on multi-rank runs).

    LT_SECTIONS=1 python -m torch.distributed.run ... -m litetorch_b200.models.run_config --config ep8

Code brackets a region with `with section("moe.route"):`; when the environment variable is unset the context manager
does nothing.  With `LT_NVTX=1` every section also opens an NVTX range of the same name, so the fused paths show up
by name on a timeline profiler.  `report()` synchronises once, sums the event pairs per name and returns {name: (calls, total ms)};
`run_config` prints it from rank 0 after the timed steps.  Sections on the same stream may nest; the times of nested
sections are included in their parents.
"""
from __future__ import annotations

import contextlib
import os
from collections import defaultdict

import torch

_ENABLED = os.environ.get("LT_SECTIONS", "") not in ("", "0")
_NVTX = os.environ.get("LT_NVTX", "") not in ("", "0")
_events = defaultdict(list)


def enabled() -> bool:
    return _ENABLED and torch.cuda.is_available()


@contextlib.contextmanager
def section(name: str):
    nvtx = _NVTX and torch.cuda.is_available()
    if nvtx:
        torch.cuda.nvtx.range_push(name)
    if not enabled():
        try:
            yield
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    try:
        yield
    finally:
        e1.record()
        _events[name].append((e0, e1))
        if nvtx:
            torch.cuda.nvtx.range_pop()


def reset() -> None:
    _events.clear()


def report() -> dict:
    if not enabled():
        return {}
    torch.cuda.synchronize()
    out = {name: (len(ev), round(sum(a.elapsed_time(b) for a, b in ev), 3)) for name, ev in _events.items()}
    return dict(sorted(out.items(), key=lambda kv: -kv[1][1]))
