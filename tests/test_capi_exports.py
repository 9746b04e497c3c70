"""CPU checks of the boundary: the library loads and exports exactly what include/vinf_b200.h declares."""
from __future__ import annotations

import re
from pathlib import Path

import pytest

from vinf_3080ti_b200 import _capi
from vinf_3080ti_b200.gguf_types import TRAITS, GGUFTensorType, row_bytes

REPO = Path(__file__).resolve().parent.parent


def declared_functions() -> set[str]:
    text = (REPO / "include" / "vinf_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(vqm_\w+)\s*\(", text))


@pytest.fixture(scope="module")
def lib():
    from vinf_3080ti_b200 import build

    build.build()
    return _capi.load()


def test_every_declared_entry_point_is_exported_and_bound(lib):
    declared = declared_functions()
    assert declared, "header parse found nothing"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/vinf_b200.h but not exported"
    assert declared == set(_capi.SIGNATURES), declared ^ set(_capi.SIGNATURES)


def test_header_type_ids_match_the_python_table():
    text = (REPO / "include" / "vinf_b200.h").read_text()
    ids = {name: int(val) for name, val in re.findall(r"VQM_(\w+) = (\d+)", text) if name in GGUFTensorType.__members__}
    assert ids == {t.name: int(t) for t in TRAITS}


def test_status_codes_map_to_the_reference_exceptions():
    assert _capi._EXC == {1: KeyError, 2: ValueError, 3: TypeError, 4: MemoryError, 5: RuntimeError}


def test_row_bytes_of_the_benchmark_shapes():
    assert row_bytes(GGUFTensorType.Q4_K, 5120) == 2880
    assert row_bytes(GGUFTensorType.Q3_K, 5120) == 2200
    assert row_bytes(GGUFTensorType.Q6_K, 5120) == 4200
    assert row_bytes(GGUFTensorType.Q4_K, 17408) == 9792
    with pytest.raises(ValueError):
        row_bytes(GGUFTensorType.Q4_K, 100)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", tmp_path / "libvinf_b200.so")
    with pytest.raises(_capi.ExtensionMissingError):
        _capi.load()
