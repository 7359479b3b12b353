"""Logging set-up.  Level from ``NANOENGINE_LOG_LEVEL`` (or the reference's ``DLENGINE_LOG_LEVEL``) or Config.log_level.
Parity: reference dlengine/logging.py, rust/src/logging.rs."""
from __future__ import annotations

import logging
import os
import sys

_FMT = "%(asctime)s %(levelname).1s %(name)s: %(message)s"


def get_logger(name: str = "nanoengine", level: str | None = None) -> logging.Logger:
    lg = logging.getLogger(name)
    if not lg.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FMT, "%H:%M:%S"))
        lg.addHandler(h)
        lg.propagate = False
    lvl = level or os.environ.get("NANOENGINE_LOG_LEVEL") or os.environ.get("DLENGINE_LOG_LEVEL") or "INFO"
    lg.setLevel(getattr(logging, lvl.upper(), logging.INFO))
    return lg
