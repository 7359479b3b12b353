"""Every operator has two bodies (CUDA and plain PyTorch) reached through one front door: their signatures must agree, or a
call that works on CPU fails on the GPU."""
import inspect

from nanoengine_b200.ops import reference as ref


def test_cuda_and_reference_bodies_take_the_same_arguments():
    import importlib
    sm100 = importlib.import_module("nanoengine_b200.ops.sm100")
    bad = []
    for name, fn in inspect.getmembers(ref, inspect.isfunction):
        if name.startswith("_") or fn.__module__ != ref.__name__:
            continue
        other = getattr(sm100, name, None)
        if other is None or other is fn or not inspect.isfunction(other):
            continue
        a, b = inspect.signature(fn).parameters, inspect.signature(other).parameters
        na, nb = [p for p in a], [p for p in b]
        # the CUDA body may take extra trailing arguments (an output buffer, a precision switch) as long as they have defaults
        extra_ok = all(b[p].default is not inspect.Parameter.empty for p in nb[len(na):])
        if len(na) > len(nb) or not extra_ok:
            bad.append((name, na, nb))
    assert not bad, bad
