"""The shared library loads without a GPU and exports every entry point the header declares."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

from alignquant_b200 import _lib

HEADER = Path(__file__).resolve().parents[1] / "include" / "alignquant_b200.h"


def declared_symbols() -> list[str]:
    text = HEADER.read_text()
    return re.findall(r"AQ_API\s+[\w\s\*]+?\b(aq_\w+)\s*\(", text)


def test_header_symbols_are_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 9 and len(set(names)) == len(names)
    lib = ctypes.CDLL(str(_lib.library_path()))
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures and header declarations differ"


def test_pure_host_entry_points():
    lib = _lib.load()
    assert lib.aq_version() >= 100
    assert lib.aq_prepared_bytes(2, 3, 4, 2) == 2048 + 4 * 2048 + 2 * 4096
    assert lib.aq_prepared_bytes(2, 3, 4, 1) < 0 and "t4 + t8" in _lib.last_error()
    assert lib.aq_linear_workspace_bytes(0, 1, 1, 0, 0) < 0
    assert lib.aq_linear_workspace_bytes(64, 4, 4, 0, 4) == 0  # explicit splits: cluster kernel, no scratch
