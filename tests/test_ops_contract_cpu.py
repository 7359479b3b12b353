"""Every operator has a CUDA body and a PyTorch body behind one front door; the bodies must agree on their parameters, or a
call that works on CPU breaks on the GPU (and the other way round).  The CUDA module is parsed, not imported: it needs no
kernel library for this check."""
import ast
import inspect
import os

from nanoengine_b200.ops import reference


def test_cuda_and_reference_bodies_share_their_leading_parameters():
    path = os.path.join(os.path.dirname(reference.__file__), "sm100.py")
    tree = ast.parse(open(path).read())
    cuda = {n.name: [a.arg for a in n.args.args] for n in tree.body if isinstance(n, ast.FunctionDef) and not n.name.startswith("_")}
    checked = 0
    for name, params in cuda.items():
        fn = getattr(reference, name, None)
        if fn is None or not callable(fn):
            continue                                   # CUDA-only helpers (pre-quantised activations, status words, ...)
        ref_params = list(inspect.signature(fn).parameters)
        n = min(len(ref_params), len(params))
        assert params[:n] == ref_params[:n], f"{name}: {params} vs {ref_params}"
        checked += 1
    assert checked >= 25
