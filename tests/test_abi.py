"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments with an error code and message before touching a device."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "b2g.h").read_text()
DECLARED = re.findall(r"^B2G_API\s+[\w\s\*]+?\b(b2g_\w+)\s*\(", HEADER, flags=re.M)


def test_header_declares_entry_points():
    assert len(DECLARED) >= 24 and len(set(DECLARED)) == len(DECLARED)


@pytest.mark.parametrize("name", DECLARED)
def test_symbol_exported(lib, name):
    assert getattr(lib, name) is not None


def test_binding_table_covers_header():
    from b2g import _lib

    assert set(_lib.SIGNATURES) == set(DECLARED)


def test_binding_argument_counts_and_kinds_match_the_header():
    """The ctypes table is written by hand: every prototype's parameter list is parsed from the header and compared with it
    (count, and pointer / 64-bit / 32-bit / float per position), so a drifted binding fails here instead of on a GPU."""
    from b2g import _lib

    protos = dict(re.findall(r"^B2G_API\s+[\w\s\*]+?\b(b2g_\w+)\s*\(([^;]*?)\)\s*;", HEADER, flags=re.M | re.S))
    assert set(protos) == set(DECLARED)

    def kind(param: str) -> str:
        param = " ".join(param.split())
        if "*" in param:
            return "ptr"
        if param.startswith("int64_t"):
            return "i64"
        if param.startswith("float"):
            return "f32"
        if param.startswith("int "):
            return "i32"
        raise AssertionError(f"unrecognised parameter {param!r}")

    table = {C.c_void_p: "ptr", C.c_char_p: "ptr", C.c_int64: "i64", C.c_int32: "i32", C.c_int: "i32", C.c_float: "f32"}
    for name, params in protos.items():
        want = [] if params.strip() in ("", "void") else [kind(p) for p in params.split(",")]
        got = [table[t] for t in _lib.SIGNATURES[name][1]]
        assert got == want, f"{name}: binding {got} != header {want}"


def test_every_entry_cites_the_reference():
    # each prototype's comment names the reference lines it replaces
    blocks = re.split(r"\n\s*\n", HEADER)
    for name in DECLARED:
        if name in ("b2g_last_error", "b2g_abi_version", "b2g_set_iq2xxs_grid") or name.endswith("_bytes"):
            continue
        block = next(b for b in blocks if re.search(rf"\b{name}\s*\(", b))
        assert re.search(r"\.py:\d+", block) or "no counterpart in the reference" in block, f"{name} lacks a reference citation"


def test_argument_errors_do_not_need_a_device(lib):
    assert lib.b2g_abi_version() == 1
    rc = lib.b2g_dequant(99, None, 1, 256, None, None)
    assert rc == -1 and b"unsupported GGUF type" in lib.b2g_last_error()
    rc = lib.b2g_dequant(12, None, 1, 100, None, None)
    assert rc == -1 and b"multiple" in lib.b2g_last_error()
    rc = lib.b2g_qlinear_fwd(12, None, None, None, None, None, None, 4, 4, 100, None, None)
    assert rc == -1 and b"K=100" in lib.b2g_last_error()
    rc = lib.b2g_router_topk(None, 0, None, 0, None, 4, 128, 8, None)
    assert rc == -1 and b"256 experts" in lib.b2g_last_error()
    rc = lib.b2g_lora_down(None, None, 0, C.c_float(1.0), None, None, 4, 128, 17, None)
    assert rc == -1 and b"rank" in lib.b2g_last_error()
    bad = (C.c_uint8 * 2048)(*([7] * 2048))
    rc = lib.b2g_set_iq2xxs_grid(bad)
    assert rc == -1 and b"8/25/43" in lib.b2g_last_error()
    assert lib.b2g_route_plan_workspace_bytes(1024, 256) >= 2 * 256 * 4
    assert lib.b2g_grouped_tiles_bytes(1024, 8) % 16 == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from b2g import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("B2G_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.B2GError, match="no CPU or PyTorch fallback"):
        _lib.load()
