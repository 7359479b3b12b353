"""Operator front door.

Every operator has exactly two bodies: the sm_100a CUDA kernel (``ops.sm100``, used for any CUDA
tensor and failing loudly when the kernel library is missing) and the plain-PyTorch statement
(``ops.reference``, used on CPU and as the numerical oracle in tests).  There is no vendor or
architecture dispatch beyond "is this tensor on the GPU".
"""
from __future__ import annotations

import torch

from . import reference

_sm100 = None


def _get_sm100():
    global _sm100
    if _sm100 is None:
        import importlib
        _sm100 = importlib.import_module(__name__ + ".sm100")
    return _sm100


def impl(t: torch.Tensor):
    return _get_sm100() if t.is_cuda else reference


def __getattr__(name):
    # ops.<fn>(first_tensor, ...) dispatches on the device of the first tensor argument
    if name.startswith("_"):
        raise AttributeError(name)
    ref_fn = getattr(reference, name, None)
    if ref_fn is None:
        raise AttributeError(name)

    if isinstance(ref_fn, type) or name == "dense":
        return ref_fn                      # value types and pure helpers are shared by both bodies

    def dispatch(*args, **kw):
        for a in args:
            if isinstance(a, reference.QAct):
                a = a.x
            if isinstance(a, torch.Tensor):
                return getattr(impl(a), name)(*args, **kw)
        return ref_fn(*args, **kw)

    dispatch.__name__ = name
    return dispatch
