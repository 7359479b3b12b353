"""In-tree build of the native parts.

Three artefacts land in ``nanoengine_b200/_native``:

* ``_core*.so``      C++20 + pybind11: scheduler, block manager, wire codec, metrics.
* ``libne_kernels.so`` CUDA sm_100a kernels with a plain C ABI (loaded with ctypes, so
  building needs neither torch headers nor a GPU; nvcc cross-compiles).
* ``ne-gateway``     C++ HTTP gateway binary.

The reference builds its native side with maturin/cargo (pyproject.toml:1-3,66-76) and
JIT-compiles CUDA through tvm_ffi (dlengine/runtime/kernel/jit/sgl/utils.py:76-123); here
everything is ahead-of-time so the shared objects travel with the source tree.

Run ``python -m nanoengine_b200.build_native`` (add ``--force`` to rebuild everything).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_native"
OBJ = OUT / "obj"
REPO = PKG.parent

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xptxas", "-v", "-DNDEBUG", "-rdc=true"] + GENCODE


def _stamp(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _needs(target: Path, stamp: str, force: bool) -> bool:
    sf = target.with_suffix(target.suffix + ".stamp")
    if force or not target.exists() or not sf.exists() or sf.read_text() != stamp:
        return True
    return False


def _mark(target: Path, stamp: str):
    target.with_suffix(target.suffix + ".stamp").write_text(stamp)


def _run(cmd, log: Path | None = None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}")
    return r


def _quiet_run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError((r.stdout + r.stderr)[-600:])
    return r


def build_core(force=False) -> Path:
    import pybind11
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    target = OUT / f"_core{suffix}"
    srcs = list((CSRC / "core").glob("*.cpp")) + list((CSRC / "core").glob("*.h"))
    stamp = _stamp(srcs)
    if _needs(target, stamp, force):
        cmd = [CXX, "-O2", "-std=c++20", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall",
               f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}",
               str(CSRC / "core" / "bindings.cpp"), "-o", str(target)]
        _run(cmd)
        _mark(target, stamp)
    return target


def build_kernels(force=False, debug_bounds=False) -> Path:
    """`debug_bounds`: the same sources with -DNE_DEBUG_BOUNDS into libne_kernels_dbg.so (kernels compare the cache rows, pages,
    state slots and expert ids they take from tables with the bounds the worker registers; loaded when NE_DEBUG_BOUNDS=1)."""
    target = OUT / ("libne_kernels_dbg.so" if debug_bounds else "libne_kernels.so")
    OBJ = OUT / ("obj_dbg" if debug_bounds else "obj")
    NVCC_FLAGS = globals()["NVCC_FLAGS"] + (["-DNE_DEBUG_BOUNDS"] if debug_bounds else [])
    kdir = CSRC / "kernels"
    cus = sorted(kdir.glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))
    hdrs = sorted(kdir.glob("*.cuh")) + sorted(kdir.glob("*.h")) + sorted((CSRC / "comm").glob("*.cuh")) + sorted((CSRC / "comm").glob("*.h"))
    if not cus:
        return target
    OBJ.mkdir(parents=True, exist_ok=True)
    hstamp = _stamp(hdrs, " ".join(NVCC_FLAGS))
    objs, jobs = [], []
    for cu in cus:
        obj = OBJ / (cu.stem + ".o")
        objs.append(obj)
        st = _stamp([cu], hstamp)
        if _needs(obj, st, force):
            jobs.append((cu, obj, st))

    def one(job):
        cu, obj, st = job
        _run([NVCC, *NVCC_FLAGS, f"-I{kdir}", f"-I{CSRC / 'comm'}", "-c", str(cu), "-o", str(obj)],
             log=OBJ / (cu.stem + ".ptxas.log"))
        _mark(obj, st)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(one, jobs))
    lstamp = _stamp(objs)
    if _needs(target, lstamp, force or bool(jobs)):
        _run([NVCC, "-shared", "-rdc=true", *GENCODE, "-o", str(target), *map(str, objs), "-lcudart"])
        _mark(target, lstamp)
    return target


def build_gateway(force=False) -> Path:
    target = OUT / "ne-gateway"
    gdir = REPO / "gateway"
    srcs = sorted(gdir.glob("*.cpp")) + sorted(gdir.glob("*.h"))
    if not srcs:
        return target
    stamp = _stamp(srcs)
    if _needs(target, stamp, force):
        _run([CXX, "-O2", "-std=c++20", "-pthread", "-Wall", *map(str, sorted(gdir.glob("*.cpp"))), "-o", str(target)])
        _mark(target, stamp)
    return target


def build_sanitized(kind: str = "address,undefined", force=False) -> dict:
    """Sanitizer builds of the host-side C++ (nothing here runs on a GPU): the control-plane exerciser
    `csrc/core/selftest.cpp` and the gateway, compiled with -fsanitize=<kind> into `_native/san/`.  `kind` is
    "address,undefined" or "thread".  The CPU test suite builds and runs both kinds."""
    tag = "tsan" if "thread" in kind else "asan"
    out = OUT / "san"
    out.mkdir(parents=True, exist_ok=True)
    flags = ["-std=c++20", "-O1", "-g", f"-fsanitize={kind}", "-fno-omit-frame-pointer", "-pthread"]

    def compile_(srcs, target):
        # the configured compiler may be a wrapper without the sanitizer runtimes: try the system ones before giving up
        last = None
        for cxx in dict.fromkeys([CXX, "/usr/bin/g++", "g++", "clang++"]):
            try:
                _quiet_run([cxx, *flags, *map(str, srcs), "-o", str(target)])
                return
            except (RuntimeError, FileNotFoundError) as e:
                last = e
        raise RuntimeError(f"no compiler here links -fsanitize={kind}: {last}")

    core_srcs = sorted((CSRC / "core").glob("*.h")) + [CSRC / "core" / "selftest.cpp"]
    selftest = out / f"core_selftest_{tag}"
    st = _stamp(core_srcs, kind)
    if _needs(selftest, st, force):
        compile_([CSRC / "core" / "selftest.cpp"], selftest)
        _mark(selftest, st)
    gdir = REPO / "gateway"
    gsrcs = sorted(gdir.glob("*.cpp")) + sorted(gdir.glob("*.h"))
    gateway = out / f"ne-gateway-{tag}"
    st = _stamp(gsrcs, kind)
    if _needs(gateway, st, force):
        compile_(sorted(gdir.glob("*.cpp")), gateway)
        _mark(gateway, st)
    return {"selftest": selftest, "gateway": gateway}


def build_all(force=False):
    OUT.mkdir(parents=True, exist_ok=True)
    (OUT / "__init__.py").touch()
    return {"core": build_core(force), "kernels": build_kernels(force), "gateway": build_gateway(force)}


if __name__ == "__main__":
    res = build_all(force="--force" in sys.argv)
    if "--debug-bounds" in sys.argv:
        res["kernels (bounds-checked)"] = build_kernels("--force" in sys.argv, debug_bounds=True)
    for k, v in res.items():
        print(f"{k}: {v} ({'ok' if Path(v).exists() else 'absent'})")
