"""Named ranges for timelines (Nsight Systems, torch.profiler): `with nvtx.range("prefill/forward"): ...`.

Off by default - a range costs two driver calls - and switched on by `NE_NVTX=1` or `enable(True)`; on CPU-only builds the
context manager does nothing.  The worker wraps the phases of a step (prepare, forward, sample, copy-back) and the engine
wraps scheduling and migration.
Parity: reference named ranges such as `nano_pp/send_hidden` (tests/test_deepseek_pp_model.py:66-71) and the torch.profiler
sessions of runtime/runner/model_runner.py:561-652.
"""
from __future__ import annotations

import contextlib
import os

_ON = os.environ.get("NE_NVTX", "0") == "1"


def enable(on: bool = True) -> None:
    global _ON
    _ON = bool(on)


def enabled() -> bool:
    return _ON


@contextlib.contextmanager
def range(name: str):
    if not _ON:
        yield
        return
    import torch
    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
