"""CPU: the C-ABI library builds, loads, exports every symbol the header declares, and
rejects bad arguments on the host without touching a GPU."""
import ctypes as C
import os
import re

import pytest

from moe_gen_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    src = open(os.path.join(ROOT, "include", "moegen_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mg_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(built_lib):
    lib = C.CDLL(built_lib)
    names = _header_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/moegen_b200.h but not exported"


def test_binding_covers_the_header(built_lib):
    declared = set(_header_functions()) - {"mg_last_error"}
    assert declared == set(L.SIGNATURES), declared ^ set(L.SIGNATURES)


def test_binding_argument_counts_match_the_header():
    """Every prototype in the header has as many parameters as the ctypes table gives its function."""
    src = open(os.path.join(ROOT, "include", "moegen_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    protos = dict(re.findall(r"\b(mg_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", src, flags=re.S))
    assert set(L.SIGNATURES) <= set(protos)
    for name, argtypes in L.SIGNATURES.items():
        params = protos[name].strip()
        n = 0 if params in ("", "void") else params.count(",") + 1
        assert n == len(argtypes), f"{name}: header declares {n} parameters, the binding passes {len(argtypes)}"


def test_layer_desc_matches_header():
    src = open(os.path.join(ROOT, "include", "moegen_b200.h")).read()
    body = re.search(r"typedef struct mg_layer_desc \{(.*?)\} mg_layer_desc;", src, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b(?:int32_t|float)\s+([a-z_0-9]+)\s*;", body)
    assert fields == [f[0] for f in L.LayerDesc._fields_]
    assert C.sizeof(L.LayerDesc) == 4 * len(fields)


@pytest.mark.parametrize("field,value,code", [
    ("hidden", 250, -2), ("inter", 100, -2), ("top_k", 0, -2), ("top_k", 65, -2),
    ("gating", 9, -3), ("weight_format", 7, -3), ("ep_size", 3, -3), ("struct_bytes", 8, -3),
])
def test_create_rejects_bad_descriptions_on_the_host(built_lib, field, value, code):
    lib = L.load()
    d = L.LayerDesc(C.sizeof(L.LayerDesc), 256, 128, 0, 64, 6, 1, 1, 0, 0, 1.0, 0, 0, 0, 1)
    setattr(d, field, value)
    h = C.c_void_p()
    assert lib.mg_create(C.byref(d), C.byref(h)) == code
    assert lib.mg_last_error() != b""
    assert not h.value


def test_null_arguments_are_errors_not_crashes(built_lib):
    lib = L.load()
    assert lib.mg_create(None, None) == -1
    assert lib.mg_destroy(None) == -5
    n = C.c_size_t()
    assert lib.mg_packed_weight_bytes(None, C.byref(n)) == -5
    assert lib.mg_dequant_fp8_block128(None, None, 1, 16, None, None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        L.load()


def test_host_chunk_schedule_covers_every_token_once():
    """forward_host's chunk sizes: they add up to T; with more than two chunks the first and last
    are half a chunk and none exceeds twice the nominal size."""
    from moe_gen_b200.layer import MoELayer
    for T in (0, 1, 100, 8192, 8193, 16384, 16385, 20000, 40000, 65536, 100001):
        for c in (128, 4096, 8192, 16384):
            sizes = MoELayer.host_chunks(T, c)
            assert sum(sizes) == T and all(n > 0 for n in sizes), (T, c, sizes)
            assert all(n <= 2 * c for n in sizes), (T, c, sizes)
            if T > 2 * c:
                assert sizes[0] == sizes[-1] == max(128, c // 2)
