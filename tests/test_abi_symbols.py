"""The C-ABI library builds, loads and exports every symbol include/turkce_b200.h declares
(no compute calls: this runs without a GPU)."""
import ctypes
import os
import re

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "turkce_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from turkce_llm_b200 import build, lib
    path = build.build()
    assert os.path.exists(path)
    names = declared_symbols()
    assert len(names) >= 30
    dll = ctypes.CDLL(path)
    missing = [n for n in names if not hasattr(dll, n)]
    assert not missing, missing
    # the Python binding declares a signature for every symbol of the header and nothing else
    assert sorted(lib.SIGNATURES) == names


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from turkce_llm_b200 import lib
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        lib.load()
    except lib.TbError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("a missing library must raise")


def test_kernels_are_blackwell_native():
    src = open(os.path.join(ROOT, "turkce_llm_b200", "csrc", "ptx.cuh")).read()
    for needle in ("tcgen05.mma", "tcgen05.alloc", "tcgen05.ld", "cp.async.bulk.tensor", "tcgen05.commit"):
        assert needle in src
    for root, _, files in os.walk(os.path.join(ROOT, "turkce_llm_b200", "csrc")):
        for f in files:
            text = open(os.path.join(root, f)).read()
            assert (".multi" + "cast::cluster") not in text, f   # no multicast loads anywhere
