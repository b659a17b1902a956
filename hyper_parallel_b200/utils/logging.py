"""Rank-aware logging and per-step metrics as JSON lines."""
from __future__ import annotations

import json
import logging
import os
import sys
import time
from typing import Optional

from ..collectives import cc


def get_logger(name: str = "hyper_parallel_b200", level: Optional[str] = None) -> logging.Logger:
    """Logger that prefixes the rank and, unless ``HPB_LOG_ALL_RANKS=1``, is silent off rank 0."""
    logger = logging.getLogger(name)
    if getattr(logger, "_hpb_configured", False):
        return logger
    lvl = (level or os.environ.get("HPB_LOG_LEVEL", "INFO")).upper()
    handler = logging.StreamHandler(sys.stderr)
    handler.setFormatter(logging.Formatter(f"%(asctime)s [rank {cc.get_rank()}] %(levelname)s %(name)s: %(message)s"))
    logger.addHandler(handler)
    logger.setLevel(lvl if (cc.get_rank() == 0 or os.environ.get("HPB_LOG_ALL_RANKS") == "1") else "ERROR")
    logger.propagate = False
    logger._hpb_configured = True
    return logger


class MetricsWriter:
    """Appends one JSON object per training step (tokens/s, MFU, loss, grad norm, ...)."""

    def __init__(self, path: Optional[str]):
        self.path = path if cc.get_rank() == 0 else None
        if self.path:
            os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)

    def write(self, step: int, **metrics) -> None:
        if not self.path:
            return
        rec = {"step": step, "time": time.time()}
        rec.update({k: (float(v) if hasattr(v, "__float__") else v) for k, v in metrics.items()})
        with open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")
