"""The ctypes declarations of the kernel library against the C definitions in the sources: a parameter too many or too
few does not fail at the call, it corrupts the arguments behind it (a pointer passed as an int loses its upper half)."""

import glob
import os
import re

from sllm_b200.ops import _lib

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "sllm_b200", "csrc")


class _Recorder:
    """Stands in for the loaded library: `_declare` sets restype and argtypes on whatever it is handed."""

    def __getattr__(self, name):
        fn = type("Fn", (), {})()
        self.__dict__[name] = fn
        return fn


def test_every_entry_point_is_declared_with_as_many_parameters_as_it_has():
    src = "".join(open(f).read() for f in sorted(glob.glob(os.path.join(CSRC, "*.cu"))))
    rec = _Recorder()
    _lib._declare(rec)
    checked = 0
    for name, fn in rec.__dict__.items():
        if not hasattr(fn, "argtypes"):
            continue
        m = re.search(r"SLLM_EXPORT\s+[\w\s\*]+?\b" + name + r"\s*\(([^)]*)\)", src)
        assert m, f"{name} is declared for ctypes but not defined in the sources"
        params = [p for p in m.group(1).split(",") if p.strip() and p.strip() != "void"]
        assert len(params) == len(fn.argtypes), f"{name}: {len(params)} parameters in C, {len(fn.argtypes)} declared"
        checked += 1
    assert checked > 40
