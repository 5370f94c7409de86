"""The C-ABI library loads and exports every symbol include/b200cp.h declares
(no compute: this runs without a GPU)."""
import ctypes
import os
import re


def test_exports_match_header(lib_built):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = open(os.path.join(root, "include", "b200cp.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(b200cp_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) >= 18
    lib = ctypes.CDLL(lib_built)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/b200cp.h but not exported"


def test_test_header_exports(lib_built):
    """The test-only header (diagnostics, test hooks) is exported and bound too, apart from the product interface."""
    from paralleltnnlayers_b200 import _lib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", "b200cp_test.h")).read(), flags=re.S)
    declared = set(re.findall(r"\b(b200cp_[a-z0-9_]+)\s*\(", hdr))
    assert declared == set(_lib.TEST_EXPORTS)
    lib = ctypes.CDLL(lib_built)
    for name in declared:
        assert hasattr(lib, name)
    assert not declared & set(_lib.EXPORTS)


def test_python_binding_covers_header(lib_built):
    from paralleltnnlayers_b200 import _lib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", "b200cp.h")).read(), flags=re.S)
    declared = set(re.findall(r"\b(b200cp_[a-z0-9_]+)\s*\(", hdr))
    assert declared == set(_lib.EXPORTS)


def test_shape_struct_layout():
    from paralleltnnlayers_b200 import TensorShape
    assert [f[0] for f in TensorShape._fields_] == ["N", "H", "W", "pad", "T", "C", "Y", "X", "Rank"]
    assert ctypes.sizeof(TensorShape) == 36


def test_argument_errors_without_gpu(lib_built):
    """Validation happens before any CUDA call: bad arguments give status codes, not crashes."""
    from paralleltnnlayers_b200 import _lib
    s = _lib.TensorShape(N=1, H=4, W=4, pad=1, T=2, C=2, Y=3, X=3, Rank=2)
    assert _lib.lib.b200cp_cp4_fwd(None, None, None, None, None, None, None, None, 0) == -1
    assert _lib.lib.b200cp_cp4_fwd(ctypes.byref(s), None, None, None, None, None, None, None, 0) == -1
    assert b"null" in _lib.lib.b200cp_last_error_string()
    z = _lib.TensorShape(N=0, H=4, W=4, pad=1, T=2, C=2, Y=3, X=3, Rank=2)
    assert _lib.lib.b200cp_cp4_bwd_filter_workspace_bytes(ctypes.byref(z), 0) == 0
    assert _lib.lib.b200cp_cp4_bwd_filter_workspace_bytes(ctypes.byref(s), 0) > 0
    assert _lib.lib.b200cp_status_string(-3) == b"workspace missing or too small"
    assert _lib.lib.b200cp_version() >= 100
