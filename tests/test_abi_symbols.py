"""CPU: the shared library loads without a GPU and exports every symbol the header declares;
the ctypes table binds exactly that set."""
import ctypes
import os
import re

from ancora_cutile_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            src = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"ANC_API\s+[\w\s\*]+?\b(anc_\w+)\s*\(", src)
    return names


def test_header_symbols_exported():
    names = _declared()
    assert len(names) >= 40
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_ctypes_table_covers_header():
    assert sorted(_declared()) == sorted(_lib.SIGNATURES)


def test_no_gpu_calls_fail_with_status_not_crash():
    l = _lib.lib()
    assert l.anc_version() >= 100
    n = ctypes.c_int(-1)
    assert l.anc_device_count(ctypes.byref(n)) == 0 and n.value >= 0
    assert l.anc_ctx_destroy(None) == 0
    assert l.anc_adamw_plan_destroy(None) == 0
    assert l.anc_muon_plan_destroy(None) == 0
    # argument validation happens before any CUDA call
    assert l.anc_adamw_step(None, None, 0, 0, 0, None) == _lib.E_INVALID
    assert b"NULL" in l.anc_last_error()


def test_product_never_reaches_the_oracle_or_torch():
    """The package is the product: it must not import the CPU oracle (test infrastructure), torch,
    triton or anything under a scratch folder, in any of its modules."""
    pkg = os.path.join(ROOT, "ancora_cutile_b200")
    bad = re.compile(r"^\s*(from|import)\s+(oracle|torch|triton|_work)\b", re.M)
    for fn in sorted(os.listdir(pkg)):
        if fn.endswith(".py"):
            assert not bad.search(open(os.path.join(pkg, fn)).read()), fn
    for fn in sorted(os.listdir(os.path.join(pkg, "csrc"))):
        src = open(os.path.join(pkg, "csrc", fn)).read()
        assert "oracle" not in src and "torch" not in src, fn


def test_missing_library_is_an_error_not_a_fallback(tmp_path, monkeypatch):
    """With no built library the loader raises; nothing computes on the host instead."""
    import pytest
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libancora_b200.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
