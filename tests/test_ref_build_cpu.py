"""The recipe that builds the reference project's own CUDA kernels as a checker (oracle/ref_build) works where the
reference tree is present, and the library exports every entry point the GPU tests bind.  No GPU call is made."""
import ctypes
import os

import pytest

from oracle.ref_build import build_ref
from tests import ref_kernels


@pytest.mark.skipif(not os.path.isdir(os.path.join(build_ref.DEFAULT_ROOT, build_ref.KERNELS)), reason="reference tree not present")
def test_reference_kernels_build_and_export():
    path = build_ref.build()
    assert path and os.path.exists(path) and path == ref_kernels.PATH
    lib = ctypes.CDLL(path)
    for name in ref_kernels._SIG:
        assert hasattr(lib, name), name


def test_nothing_of_the_reference_is_copied():
    """The recipe compiles the reference's files in place: this repository holds only the entry points and a stub header."""
    here = os.path.dirname(build_ref.__file__)
    files = sorted(os.path.relpath(os.path.join(d, f), here) for d, _, fs in os.walk(here) for f in fs if "__pycache__" not in d)
    assert files == ["__init__.py", "build_ref.py", "raf_ref_entry.cu", "stub/raf/device.h"]
