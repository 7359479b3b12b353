"""Sanitizer builds of the host-side C++: the control-plane exerciser (scheduler, block pool, slot pools, L3 index, wire codec)
and the HTTP gateway, under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer.  These stand in for the
device-side memory checker, which is not available where the GPU tests run: the kernels are covered by the fp32-oracle tests,
the code that feeds them indices and tables is covered here."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(kind):
    from nanoengine_b200.build_native import build_sanitized
    try:
        return build_sanitized(kind)
    except RuntimeError as e:                      # a toolchain without the sanitizer runtime
        pytest.skip(f"cannot build with -fsanitize={kind}: {e}")


@pytest.mark.parametrize("kind", ["address,undefined", "thread"])
def test_control_plane_selftest_is_clean(kind):
    exe = _build(kind)["selftest"]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1",
               TSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    if "thread" in kind and r.returncode != 0 and "unexpected memory mapping" in r.stderr:
        pytest.skip("ThreadSanitizer cannot map its shadow memory in this container")
    assert r.returncode == 0 and "selftest ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    assert "runtime error" not in r.stderr and "Sanitizer" not in r.stderr, r.stderr[-4000:]


def test_gateway_scenarios_under_address_sanitizer():
    """The gateway's own scenario tests, run against the instrumented binary."""
    exe = _build("address,undefined")["gateway"]
    env = dict(os.environ, NE_GATEWAY_BIN=str(exe), ASAN_OPTIONS="detect_leaks=0", UBSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gateway.py"), "-x", "-q", "-p", "no:cacheprovider"],
                       capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
