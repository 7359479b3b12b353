"""Side streams by role: one CUDA stream per (role, device, priority), created on first use and shared by every layer that plays
that role (the shared-expert branch of a MoE layer, a draft chain, ...).  A layer asks by name instead of creating streams of its
own, so 61 layers share one stream and a CUDA graph captured over them forks and joins the same one.
Parity: reference runtime/stream_pool.py (`get_cuda_stream`)."""
from __future__ import annotations

import threading
from typing import Dict, Tuple, Union

import torch

_POOL: Dict[Tuple[str, int, int], "torch.cuda.Stream"] = {}
_LOCK = threading.Lock()


def _index(device: Union[int, str, torch.device, None]) -> int:
    if device is None:
        return torch.cuda.current_device()
    if isinstance(device, int):
        return device
    d = torch.device(device)
    return torch.cuda.current_device() if d.index is None else d.index


def get_cuda_stream(role: str, device: Union[int, str, torch.device, None] = None, priority: int = 0) -> "torch.cuda.Stream":
    key = (str(role), _index(device), int(priority))
    with _LOCK:
        s = _POOL.get(key)
        if s is None:
            s = _POOL[key] = torch.cuda.Stream(device=key[1], priority=key[2])
        return s


def clear_cuda_stream_pool() -> None:
    """Forget every stream (tests; a process that switches devices wholesale)."""
    with _LOCK:
        _POOL.clear()
