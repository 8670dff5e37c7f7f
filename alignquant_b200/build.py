"""Build recipe of ``libalignquant_b200.so`` (nvcc, sm_100a only, in-tree output)."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIB_PATH = PACKAGE_DIR / "libalignquant_b200.so"
SOURCES = ("aq_abi.cu", "aq_quantize.cu", "aq_repack.cu", "aq_stream.cu", "aq_cluster_decode.cu", "aq_direct_decode.cu", "aq_decode.cu", "aq_gemm_tmem.cu", "aq_allreduce.cu", "aq_peak.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
)


def find_nvcc() -> str:
    for candidate in (
        os.environ.get("ALIGNQUANT_NVCC"),
        shutil.which("nvcc"),
        str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"),
    ):
        if candidate and Path(candidate).is_file():
            return candidate
    raise RuntimeError("nvcc not found; set ALIGNQUANT_NVCC or CUDA_HOME")


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / name for name in SOURCES] + sorted(CSRC.glob("*.cuh")) + [PACKAGE_DIR.parent / "include" / "alignquant_b200.h"]
    return any(dep.stat().st_mtime > built for dep in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source of the package into one shared library."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    build_dir = PACKAGE_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    objects = []
    procs = []
    for name in SOURCES:
        obj = build_dir / (Path(name).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / name), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    for name, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            print(f"--- {name}\n{out}")
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}")
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *objects, "-Xcompiler", "-fPIC", "-lcudart"]
    subprocess.check_call(link)
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build_library(force=True, verbose="-v" in sys.argv))
