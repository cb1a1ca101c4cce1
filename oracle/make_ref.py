"""Recipe for the live reference oracle (test infrastructure only).

``python oracle/make_ref.py [<reference checkout>]`` prepares ``oracle/_ref/``:

* the reference's ``community_kv`` Python package (its Triton decode kernels
  ``community_kv/attention/kernels/{centroid_selection,segmented_attention}.py``
  are plain Python that Triton compiles for the GPU it runs on, so they run on
  sm_100 unchanged), placed there as an importable package, exactly the files a
  ``pip install --target`` of the reference would place;
* the reference's native selector (``community_kv/attention/kernels/_csrc/
  descriptor_selection.cu`` + ``bindings.cpp``), compiled from where the sources
  lie with ``torch.utils.cpp_extension.load`` for sm_100a into
  ``_ref/community_kv/attention/kernels/_selection_native.so`` (the module name the
  reference imports, ``centroid_selection.py:470``).

Nothing under ``_ref/`` is tracked, and nothing outside ``tests/`` may import it: it
is the checker for the parity tests that run the reference's own kernels and this
library on identical inputs on the same GPU.  The patched FlashAttention prefill
kernel is not part of it (its sources are not in the reference checkout and it
only builds for sm_90).

The build needs no GPU (nvcc cross-compiles).  If the selector does not compile the
Python half is still prepared and the reason is written to ``_ref/BUILD_LOG.txt``.
"""

from __future__ import annotations

import os
import shutil
import sys
import traceback
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
# default: a checkout named "reference" beside this repository, or $CKV_REFERENCE_CHECKOUT
DEFAULT_CHECKOUT = Path(os.environ.get("CKV_REFERENCE_CHECKOUT", HERE.parents[1] / "reference"))


def _copy_package(checkout: Path) -> None:
    source = checkout / "community_kv"
    destination = TARGET / "community_kv"
    if destination.exists():
        shutil.rmtree(destination)
    shutil.copytree(
        source,
        destination,
        ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "_csrc", "*.so"),
    )
    for path in [destination, *destination.rglob("*")]:  # the checkout may be read-only
        path.chmod(0o755 if path.is_dir() else 0o644)


def _build_selector(checkout: Path) -> str:
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils import cpp_extension

    csrc = checkout / "community_kv/attention/kernels/_csrc"
    build_dir = TARGET / "build_selection_native"
    build_dir.mkdir(parents=True, exist_ok=True)
    cpp_extension.load(
        name="_selection_native",
        sources=[str(csrc / "bindings.cpp"), str(csrc / "descriptor_selection.cu")],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=["-O3", "-std=c++17", "--use_fast_math", "-lineinfo"],
        build_directory=str(build_dir),
        verbose=False,
        is_python_module=False,  # compile and link only; the tests import it on the GPU box
    )
    built = build_dir / "_selection_native.so"
    if not built.exists():
        raise RuntimeError(f"{built} was not produced")
    destination = TARGET / "community_kv/attention/kernels/_selection_native.so"
    shutil.copy2(built, destination)
    return str(destination)


def _up_to_date(checkout: Path) -> bool:
    built = TARGET / "community_kv/attention/kernels/_selection_native.so"
    if not built.exists():
        return False
    sources = list((checkout / "community_kv").rglob("*.py"))
    sources += list((checkout / "community_kv/attention/kernels/_csrc").glob("*"))
    return all(path.stat().st_mtime <= built.stat().st_mtime for path in sources)


def make(checkout: Path = DEFAULT_CHECKOUT, *, force: bool = False) -> bool:
    """Returns True when the package and the native selector are both in place."""

    if not (checkout / "community_kv").is_dir():
        raise FileNotFoundError(f"{checkout} holds no community_kv package")
    if not force and _up_to_date(checkout):
        return True
    TARGET.mkdir(exist_ok=True)
    _copy_package(checkout)
    log = TARGET / "BUILD_LOG.txt"
    try:
        path = _build_selector(checkout)
        log.write_text(f"selector built: {path}\n")
        return True
    except Exception:  # noqa: BLE001 - the Triton half is still usable
        log.write_text("selector NOT built:\n" + traceback.format_exc())
        return False


if __name__ == "__main__":
    arguments = [a for a in sys.argv[1:] if a != "--force"]
    where = Path(arguments[0]) if arguments else DEFAULT_CHECKOUT
    ok = make(where, force="--force" in sys.argv)
    print((TARGET / "BUILD_LOG.txt").read_text())
    sys.exit(0 if ok else 1)
