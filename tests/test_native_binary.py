"""Runs the native C++ test binary (csrc/test/main.cpp): C++ layers and the public C API without Python in between."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_native_cases_pass():
    exe = os.path.join(ROOT, "csrc", "test", "mf_native_tests")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-j8"], cwd=ROOT, stdout=subprocess.DEVNULL)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
    assert "0 failed" in out.stdout
