"""Loads the in-tree native extension; builds it first when it is missing and a toolchain is present."""
import importlib
import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)


def _built() -> bool:
    has_core = os.path.exists(os.path.join(_HERE, "lib", "libmf_core.so"))
    has_mod = any(f.startswith("_pymf") and f.endswith(".so") for f in os.listdir(_HERE))
    return has_core and has_mod


def build(jobs: int = 8) -> None:
    """Compile libmf_core.so and the _pymf extension in-tree (make; nvcc for sm_100a)."""
    subprocess.check_call(["make", "-j", str(jobs)], cwd=_ROOT, stdout=subprocess.DEVNULL)


if not _built():
    if os.path.exists(os.path.join(_ROOT, "Makefile")):
        build()
    else:
        raise ImportError("memfabric_hybrid_b200: native extension not built and no Makefile found")

_pymf = importlib.import_module("memfabric_hybrid_b200._pymf")
sys.modules.setdefault("memfabric_hybrid_b200._native", _pymf)
