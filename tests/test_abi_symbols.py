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


def test_options_are_validated_and_read_back():
    """Process-wide options: set, read back, reject values outside their range (no GPU involved)."""
    lib = _lib.load()
    defaults = {
        _lib.AQ_OPT_PEER_POLL_LIMIT: 1 << 22, _lib.AQ_OPT_GEMM_ROUNDING: 0, _lib.AQ_OPT_GEMM_TILE: 0,
        _lib.AQ_OPT_GEMM_SPLIT: 0, _lib.AQ_OPT_DECODE_KERNEL: 0, _lib.AQ_OPT_QUANT_FUSION_TILES: 2400,
    }
    for option, value in defaults.items():
        assert lib.aq_get_option(option) == value
    changes = {
        _lib.AQ_OPT_PEER_POLL_LIMIT: 4096, _lib.AQ_OPT_GEMM_ROUNDING: 1, _lib.AQ_OPT_GEMM_TILE: 4,
        _lib.AQ_OPT_GEMM_SPLIT: 3, _lib.AQ_OPT_DECODE_KERNEL: _lib.AQ_DECODE_KERNEL_STREAMK, _lib.AQ_OPT_QUANT_FUSION_TILES: 0,
    }
    try:
        for option, value in changes.items():
            assert lib.aq_set_option(option, value) == 0, _lib.last_error()
            assert lib.aq_get_option(option) == value
        for option, bad in ((_lib.AQ_OPT_PEER_POLL_LIMIT, 1), (_lib.AQ_OPT_GEMM_ROUNDING, 2), (_lib.AQ_OPT_GEMM_TILE, 3),
                            (_lib.AQ_OPT_GEMM_SPLIT, 9), (_lib.AQ_OPT_DECODE_KERNEL, 3), (_lib.AQ_OPT_QUANT_FUSION_TILES, -1), (99, 0)):
            assert lib.aq_set_option(option, bad) < 0
        assert lib.aq_get_option(99) < 0
    finally:
        for option, value in defaults.items():
            assert lib.aq_set_option(option, value) == 0

