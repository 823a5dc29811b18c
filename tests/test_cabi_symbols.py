"""The C-ABI library loads and exports every symbol include/caifq.h declares (no compute, no GPU)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "caifq.h")).read()
    return sorted(set(re.findall(r"CAIFQ_API[^;(]*?\b(caifq_\w+)\s*\(", text)))


def _ensure_built():
    path = os.path.join(ROOT, "caif_b200", "libcaifq.so")
    if not os.path.exists(path):
        from caif_b200 import build

        build.build()
    return path


def test_header_declares_entry_points():
    names = _declared()
    assert len(names) >= 20
    for must in ("caifq_linear_fwd", "caifq_linear_dx", "caifq_quantize_int4_per_group", "caifq_lora_linear_bwd",
                 "caifq_moe_build_dispatch", "caifq_grouped_expert_fwd"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_ensure_built())
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_matches_header():
    from caif_b200 import native

    assert sorted(native.exported_names()) == _declared()
    native.lib()  # sets argtypes on every symbol; raises if one is absent
    assert native.lib().caifq_version().decode().startswith("caifq")


def test_argument_errors_are_reported_without_a_gpu():
    from caif_b200 import native

    lib = native.lib()
    w = native.CWeight(None, None, native.I8, 0, 128, 16, 16)
    rc = lib.caifq_linear_fwd(ctypes.byref(w), None, native.F32, 4, None, native.F32, native.F32, None)
    assert rc == 1
    assert b"weight not loaded" in lib.caifq_last_error()
    rc = lib.caifq_quantize_int4_per_group(None, None, None, 16, 0, None)
    assert rc == 1
    assert b"group_size" in lib.caifq_last_error()


def test_missing_library_is_loud(tmp_path, monkeypatch):
    from caif_b200 import native

    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setattr(native, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        native.lib()
    except native.CaifqError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("expected CaifqError")
