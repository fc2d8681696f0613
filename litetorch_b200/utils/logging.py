"""Rank-prefixed logger with levels and a JSON-lines writer for per-step metrics.

The reference prints banners with std::cout and warnings with std::cerr (src/core/backend.cpp:351-359) and its training
scripts print tables (train_cat_dog.py:312-323); there are no levels and no structured metrics.  Here:

    log = get_logger()                       # "[rank 3] 12:00:01 INFO  message"; level from LT_LOG_LEVEL (default INFO)
    log.info("step %d loss %.4f", i, loss)

    mw = MetricsWriter("metrics.jsonl")      # one JSON object per line, written by rank 0 only unless all_ranks=True
    mw.write(step=i, loss=loss, tokens_per_s=tps, step_ms=ms, exposed_comm_ms=c)
    mw.close()

`MetricsWriter.write` adds the wall-clock time, the rank and, on a GPU, the allocator's high-water mark.
"""
from __future__ import annotations

import json
import logging
import os
import sys
import time
from typing import Optional

_LEVELS = {"DEBUG": logging.DEBUG, "INFO": logging.INFO, "WARNING": logging.WARNING, "WARN": logging.WARNING,
           "ERROR": logging.ERROR}


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


def get_logger(name: str = "litetorch_b200", level: Optional[str] = None, stream=None) -> logging.Logger:
    log = logging.getLogger(name)
    lvl = _LEVELS.get((level or os.environ.get("LT_LOG_LEVEL", "INFO")).upper(), logging.INFO)
    log.setLevel(lvl)
    if not getattr(log, "_lt_configured", False) or stream is not None:
        for h in list(log.handlers):
            log.removeHandler(h)
        h = logging.StreamHandler(stream or sys.stderr)
        h.setFormatter(logging.Formatter("[rank %d] %%(asctime)s %%(levelname)-5s %%(message)s" % _rank(), "%H:%M:%S"))
        log.addHandler(h)
        log.propagate = False
        log._lt_configured = True
    return log


class MetricsWriter:
    def __init__(self, path: str, all_ranks: bool = False):
        self.rank = _rank()
        self.active = all_ranks or self.rank == 0
        if all_ranks and self.rank != 0:
            root, ext = os.path.splitext(path)
            path = "%s.rank%d%s" % (root, self.rank, ext)
        self.path = path
        self._f = open(path, "a") if self.active else None

    def write(self, **metrics) -> None:
        if not self.active:
            return
        rec = {"time": round(time.time(), 3), "rank": self.rank}
        rec.update(metrics)
        try:
            import torch
            if torch.cuda.is_available() and torch.cuda.is_initialized():
                rec.setdefault("max_memory_allocated_mb", round(torch.cuda.max_memory_allocated() / 2 ** 20, 1))
        except Exception:                      # metrics must never take a training run down
            pass
        self._f.write(json.dumps(rec, default=float) + "\n")
        self._f.flush()

    def close(self) -> None:
        if self._f is not None:
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


__all__ = ["get_logger", "MetricsWriter"]
