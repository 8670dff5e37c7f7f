"""ctypes binding of ``libalignquant_b200.so`` (the C ABI in ``include/alignquant_b200.h``)."""

from __future__ import annotations

import ctypes
import os
from functools import lru_cache
from pathlib import Path

AQ_OK = 0
AQ_F16, AQ_BF16, AQ_F32 = 0, 1, 2
AQ_SCALE_TILE, AQ_SCALE_TOKEN = 0, 1
AQ_OPT_PEER_POLL_LIMIT, AQ_OPT_GEMM_ROUNDING, AQ_OPT_GEMM_TILE, AQ_OPT_GEMM_SPLIT, AQ_OPT_DECODE_KERNEL = 1, 2, 3, 4, 5
AQ_OPT_QUANT_FUSION_TILES = 6
AQ_DECODE_KERNEL_AUTO, AQ_DECODE_KERNEL_CLUSTER, AQ_DECODE_KERNEL_STREAMK = 0, 1, 2
AQ_GEMM_ROUNDING_FUSED, AQ_GEMM_ROUNDING_SEPARATE = 0, 1
GEMM_TILES = {"auto": 0, "paired": 1, "narrow": 2, "wide": 4}
SCHEDULE_CODES = {"auto": 0, "forced_decode": 1, "forced_prefill": 2, "forced_prefill_m64": 3}

_P = ctypes.c_void_p
_I32 = ctypes.c_int32
_I64 = ctypes.c_int64
_INT = ctypes.c_int

# name -> (restype, argtypes); one entry per declaration in include/alignquant_b200.h
SIGNATURES = {
    "aq_version": (_INT, []),
    "aq_last_error": (ctypes.c_char_p, []),
    "aq_quantize_act": (_INT, [_P, _INT, _I64, _I64, _P, _INT, _P, _P, _P]),
    "aq_rmsnorm_quantize": (_INT, [_P, _INT, _I64, _I64, _P, ctypes.c_float, _P, _P, _P, _P]),
    "aq_prepared_bytes": (_I64, [_I32, _I32, _I64, _I64]),
    "aq_repack": (_INT, [_P, _P, _P, _P, _P, _P, _P, _I32, _I32, _I64, _I64, _P, _I64, _P]),
    "aq_linear_workspace_bytes": (_I64, [_I64, _I32, _I32, _INT, _INT]),
    "aq_linear": (_INT, [_P, _P, _INT, _I64, _P, _I32, _I32, _P, _INT, _INT, _INT, _P, _P, _I64, _P, _P]),
    "aq_set_option": (_INT, [_INT, _I64]),
    "aq_get_option": (_I64, [_INT]),
    "aq_linear_ahead": (_INT, [_P, _P, _INT, _I64, _P, _I32, _I32, _P, _INT, _INT, _INT, _P, _P, _I64, _P, _P, _I64, _P]),
    "aq_linear_decode_static": (_INT, [_P, _P, _INT, _I64, _P, _I32, _I32, _P, _INT, _P, _P]),
    "aq_linear_plan": (_INT, [_I64, _I32, _I32, _INT, _INT, _P, _P, _P]),
    "aq_allreduce_buffer_bytes": (_I64, [_I32, _I64]),
    "aq_allreduce_f32": (_INT, [_P, _P, _I64, _I32, _I32, _P, _I64, _P]),
    "aq_linear_allreduce": (_INT, [_P, _P, _INT, _I64, _P, _I32, _I32, _P, _INT, _P, _I32, _I32, _P, _I64, _P, _I64, _P]),
    "aq_quant_linear": (_INT, [_P, _INT, _I64, _P, _I32, _I32, _P, _INT, _P, _P, _P, _P, _I64, _I32, _I32, _P, _I64, _P, _I64, _P]),
    "aq_quant_linear_fused": (_INT, [_I64, _I32, _I32]),
    "aq_measure_int8_peak": (_INT, [_I32, _P, _P]),
    "aq_device_status": (_INT, [_P]),
}


def library_path() -> Path:
    override = os.environ.get("ALIGNQUANT_B200_LIB")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / "libalignquant_b200.so"


@lru_cache(maxsize=1)
def load() -> ctypes.CDLL:
    """Load the native library; there is no fallback path when it is missing."""
    path = library_path()
    if not path.is_file():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m alignquant_b200.build` "
            "(nvcc, sm_100a). alignquant_b200 has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def last_error() -> str:
    return load().aq_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raise ``RuntimeError`` for a non-zero status, as the reference's TORCH_CHECKs do."""
    if status != AQ_OK:
        raise RuntimeError(f"alignquant_b200: {last_error()} (status {status})")
