"""Ahead-of-time build of the native extension for sm_100a.

The reference compiles a host extension with ``torch.utils.cpp_extension.load`` and JIT-compiles
its kernels through a third-party JIT (nano_ep/backends/_build.py:24-48, csrc/jit.cpp).  Here every
kernel is compiled ahead of time into one in-tree shared object: geometry (H, K, R, L) is a run-time
argument of the kernels, so no per-shape compilation exists and nothing is compiled on first use.

``python -m nanoep_b200.utils.build`` builds; ``load_extension()`` imports the built module and only
rebuilds when the sources changed (content hash) or the shared object is missing.
"""

from __future__ import annotations

import functools
import hashlib
import importlib.util
import os
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent.parent
REPO_CSRC = PACKAGE_DIR.parent / "csrc"
BUNDLED_CSRC = PACKAGE_DIR / "_csrc"
EXT_DIR = PACKAGE_DIR / "_ext"
EXT_NAME = "nanoep_b200_C"

SOURCES = (
    "bindings.cpp",
    "pipeline.cpp",
    "gemm_bindings.cpp",
    "peer_window.cu",
    "ep_kernels.cu",
    "grouped_gemm_sm100.cu",
    "grouped_gemm_sm100_2cta.cu",
)

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def source_dir() -> Path:
    """``csrc`` of a checkout, or the copy bundled into an installed wheel."""
    for candidate in (REPO_CSRC, BUNDLED_CSRC):
        if (candidate / "bindings.cpp").exists():
            return candidate
    raise FileNotFoundError("nanoep_b200 native sources not found")


def sources_hash(extra: tuple[str, ...] = ()) -> str:
    h = hashlib.sha256()
    root = source_dir()
    for path in sorted(root.rglob("*")):
        if path.suffix in {".cu", ".cuh", ".cpp", ".hpp", ".h"}:
            h.update(path.name.encode())
            h.update(path.read_bytes())
    for item in extra:
        h.update(item.encode())
    return h.hexdigest()


def _stamp_path() -> Path:
    return EXT_DIR / f"{EXT_NAME}.stamp"


def _so_path() -> Path:
    return EXT_DIR / f"{EXT_NAME}.so"


def _import_built():
    spec = importlib.util.spec_from_file_location(EXT_NAME, _so_path())
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[EXT_NAME] = module
    return module


def build_extension(verbose: bool | None = None, force: bool = False):
    """Compile (if needed) and import the extension."""
    import torch  # noqa: F401  (must be imported before the extension's shared object)
    from torch.utils import cpp_extension

    if verbose is None:
        verbose = os.environ.get("NANOEP_BUILD_VERBOSE") == "1"
    EXT_DIR.mkdir(exist_ok=True)
    digest = sources_hash()
    if not force and _so_path().exists() and _stamp_path().exists() and _stamp_path().read_text().strip() == digest:
        return _import_built()
    root = source_dir()
    module = cpp_extension.load(
        name=EXT_NAME,
        sources=[str(root / s) for s in SOURCES],
        extra_include_paths=[str(root)],
        extra_cflags=["-O2", "-std=c++17"],
        extra_cuda_cflags=["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", *ARCH_FLAGS],
        extra_ldflags=["-lcuda", "-lstdc++", "-lm"],
        build_directory=str(EXT_DIR),
        with_cuda=True,
        verbose=verbose,
    )
    _stamp_path().write_text(digest)
    return module


@functools.cache
def load_extension():
    """Import the native module, building it first when it is missing or stale."""
    return build_extension()


def main():
    import argparse

    parser = argparse.ArgumentParser(description="Build the nanoep_b200 native extension for sm_100a")
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    module = build_extension(verbose=args.verbose or None, force=args.force)
    print(f"built {module.__file__ if hasattr(module, '__file__') else _so_path()}")


if __name__ == "__main__":
    main()


def build_all(verbose: bool | None = None, force: bool = False):
    """Build every native artefact of the package (the extension and the stand-alone C libraries)."""
    module = build_extension(verbose=verbose, force=force)
    build_noalloc(force=force)
    return module


NOALLOC_LIB = "libnep_noalloc.so"


def build_noalloc(force: bool = False) -> Path:
    """Compile the stand-alone C library with the allocation-free entry point (plain nvcc, no torch)."""
    import subprocess

    EXT_DIR.mkdir(exist_ok=True)
    src = source_dir() / "noalloc" / "plan_rows_noalloc.cu"
    out = EXT_DIR / NOALLOC_LIB
    stamp = EXT_DIR / (NOALLOC_LIB + ".stamp")
    digest = hashlib.sha256(src.read_bytes() + (src.parent / "plan_rows_noalloc.h").read_bytes()).hexdigest()
    if not force and out.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return out
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "--compiler-options", "-fPIC", "-shared", "-cudart", "shared", str(src), "-o", str(out)]
    subprocess.run(cmd, check=True)
    stamp.write_text(digest)
    return out
