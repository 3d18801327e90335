"""The shared library loads without a GPU and exports every function include/hipattn.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "hipattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hipattn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from hip_attention_b200 import _lib
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/hipattn.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype"
    assert sorted(_lib.SYMBOLS) == names
    assert lib.hipattn_abi_version() == _lib.ABI_VERSION


def test_struct_layouts_match_header_field_order():
    """ctypes structures list the header's fields in the header's order."""
    from hip_attention_b200 import _lib
    text = open(os.path.join(ROOT, "include", "hipattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for cname, cls in (("hipattn_tokens", _lib.Tokens), ("hipattn_scan_params", _lib.ScanParams),
                       ("hipattn_bsa_params", _lib.BsaParams)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s_t;" % (cname, cname), text, flags=re.S).group(1)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = decl.split(None, 1)[1] if not decl.startswith("const") else decl.split(None, 2)[2]
            for nm in names.split(","):
                fields.append(nm.strip().lstrip("*").strip())
        assert fields == [f[0] for f in cls._fields_], cname


def test_score_encoding_is_order_preserving():
    from hip_attention_b200 import _lib
    lib = _lib.load()
    import numpy as np
    vals = [float(np.float32(x)) for x in (-3.4e38, -32000.0, -1.5, -0.0, 0.0, 1e-30, 0.25, 7.0, 3.4e38)]
    codes = [lib.hipattn_encode_score(v) for v in vals]
    assert codes == sorted(codes)
    for v in vals:
        assert lib.hipattn_decode_score(lib.hipattn_encode_score(v)) == v


def test_entry_points_reject_bad_arguments_without_a_gpu():
    """Validation happens before any launch, so it can be exercised on a CPU-only box."""
    from hip_attention_b200 import _lib
    lib = _lib.load()
    assert lib.hipattn_scan_stage(None, None) == 1
    assert b"null" in lib.hipattn_error_string()
    sp = _lib.ScanParams()
    assert lib.hipattn_scan_stage(ctypes.byref(sp), None) == 1
    assert lib.hipattn_bsa_attention(None, None) == 1
    assert lib.hipattn_select_stage(None, None, 1, 4, 2, 0, 8, 4, None, None, None, None) == 1
    assert lib.hipattn_merge_partials(None, None, 1, 1, 64, 0, None, 64, None, None) == 1


def test_operator_fails_loudly_without_library(monkeypatch):
    from hip_attention_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libhipattn_sm100.so")
    with pytest.raises(_lib.HipAttnError):
        _lib.load()
