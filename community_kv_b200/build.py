"""In-tree build of the CUDA library (``libckv_b200.so``) for sm_100a.

``python -m community_kv_b200.build`` compiles every ``.cu`` file under
``csrc/`` with nvcc into one shared object next to this file.  nvcc cross
compiles without a GPU, so the build also serves as the CPU-side build check.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIBRARY_PATH = PACKAGE_DIR / "libckv_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    candidate = os.environ.get("CKV_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(candidate).exists():
        raise RuntimeError("nvcc was not found; set CKV_NVCC")
    return candidate


def sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def is_stale() -> bool:
    if not LIBRARY_PATH.exists():
        return True
    built = LIBRARY_PATH.stat().st_mtime
    inputs = list(CSRC_DIR.glob("*.cu")) + list(CSRC_DIR.glob("*.cuh"))
    inputs.append(PACKAGE_DIR.parent / "include" / "ckv_b200.h")
    return any(path.stat().st_mtime > built for path in inputs if path.exists())


def build(*, force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""

    if not force and not is_stale():
        return LIBRARY_PATH
    command = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        command += ["-Xptxas", "-v"]
    command += ["-o", str(LIBRARY_PATH), *[str(path) for path in sources()]]
    completed = subprocess.run(command, capture_output=True, text=True)
    if completed.returncode != 0:
        raise RuntimeError(
            "nvcc failed:\n" + " ".join(command) + "\n" + completed.stdout + completed.stderr
        )
    if verbose:
        sys.stderr.write(completed.stderr)
    return LIBRARY_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
