"""The header-only C++ mirror of the reference's host API (include/b200cp.hpp), compiled with g++ and run."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_cpp_mirror_of_the_reference_api():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "tests", "cpp"))
    import build as cpp_build
    exe = cpp_build.build()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.startswith("OK")
