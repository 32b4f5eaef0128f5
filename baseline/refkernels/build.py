"""Build the reference-kernel comparison extension (a measuring aid; see jit_standin.cu).

    python baseline/refkernels/build.py [--skip-peer-device-checks]

Copies the reference's Python package and native sources, unmodified, from the mounted checkout into the git-ignored
``baseline/_ref/`` and compiles its host runtime (bindings.cpp, peer.cu, pipeline.cu, dispatch_epilogue.cpp,
combine_epilogue.cpp) together with ``jit_standin.cu`` (which replaces only the reference's jit.cpp) for sm_100a.
``load()`` imports the result; ``reference_package()`` returns the reference's ``nano_ep`` module wired to it.
"""

from __future__ import annotations

import importlib
import importlib.util
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE.parent / "_ref"
BUILD_DIR = REF_OUT / "build"
NAME = "nano_ep_native"
SOURCES = ("bindings.cpp", "peer.cu", "pipeline.cu", "dispatch_epilogue.cpp", "combine_epilogue.cpp")


def stage_reference(checkout: Path) -> None:
    """Unmodified copies of the reference's package and native sources (the GPU box has no mounted checkout)."""
    for name in ("nano_ep", "csrc"):
        target = REF_OUT / name
        if target.exists():
            shutil.rmtree(target)
        shutil.copytree(checkout / name, target, ignore=shutil.ignore_patterns("__pycache__"))


PEER_CHECK_BEGIN = "            cudaPointerAttributes attributes{};"
PEER_CHECK_END = "rank \", peer, \"'s GPU \", attributes.device);\n"


def drop_peer_device_checks() -> None:
    """The one edit to the staged copy, and only when asked for (--skip-peer-device-checks).

    The reference looks up the owner of an IPC-mapped peer pointer with cudaPointerGetAttributes and refuses to go on
    when it equals the importing device (csrc/peer.cu:114-125).  With the CUDA 12.9 runtime and driver of this pool that
    call names the importing device for every mapped peer pointer, so the unmodified check stops every run on two or
    more GPUs with "Ranks must use distinct GPUs" although the ranks do sit on distinct GPUs.  The three checks that
    depend on that lookup are removed from the staged copy; nothing else of peer.cu changes."""
    path = REF_OUT / "csrc" / "peer.cu"
    text = path.read_text()
    begin = text.index(PEER_CHECK_BEGIN)
    end = text.rindex(PEER_CHECK_END, begin, text.index("auto host_addresses")) + len(PEER_CHECK_END)
    path.write_text(text[:begin] + "            // (device checks removed by baseline/refkernels/build.py --skip-peer-device-checks)\n" + text[end:])
    (REF_OUT / "PEER_CHECKS_REMOVED").write_text("peer.cu:114-125 removed from the staged copy\n")


def build(checkout: Path | None = None, verbose: bool = False, skip_peer_device_checks: bool = False):
    import torch  # noqa: F401
    from torch.utils import cpp_extension

    if checkout is None:
        # where the reference checkout is mounted: NANOEP_REFERENCE_CHECKOUT, else a sibling "reference" of the repository
        checkout = Path(os.environ.get("NANOEP_REFERENCE_CHECKOUT", HERE.parent.parent.parent / "reference"))
    if not (checkout / "csrc" / "pipeline.cu").exists():
        raise FileNotFoundError(f"no reference checkout at {checkout}; set NANOEP_REFERENCE_CHECKOUT")
    REF_OUT.mkdir(parents=True, exist_ok=True)
    marker = REF_OUT / "PEER_CHECKS_REMOVED"
    if marker.exists():
        marker.unlink()
    stage_reference(checkout)
    if skip_peer_device_checks:
        drop_peer_device_checks()
    BUILD_DIR.mkdir(exist_ok=True)
    csrc = REF_OUT / "csrc"
    return cpp_extension.load(
        name=NAME,
        sources=[str(csrc / s) for s in SOURCES] + [str(p) for p in sorted(HERE.glob("*.cu"))],
        extra_include_paths=[str(csrc), str(csrc / "include"), str(HERE)],
        extra_cflags=["-O2", "-std=c++20", "-DUSE_CUDA"],
        extra_cuda_cflags=["-O2", "-std=c++20", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a"],
        extra_ldflags=["-ldl"],
        build_directory=str(BUILD_DIR),
        with_cuda=True,
        verbose=verbose,
    )


def load():
    """Import the built extension (no compilation; raises if it was never built)."""
    import torch  # noqa: F401

    so = BUILD_DIR / f"{NAME}.so"
    if not so.exists():
        raise FileNotFoundError(f"{so} is missing: run python baseline/refkernels/build.py where the reference checkout is mounted")
    spec = importlib.util.spec_from_file_location(NAME, so)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def reference_package():
    """The reference's own ``nano_ep`` package (unmodified copy), with its extension loader pointed at the build above."""
    native = load()
    if str(REF_OUT) not in sys.path:
        sys.path.insert(0, str(REF_OUT))
    build_module = importlib.import_module("nano_ep.backends._build")
    build_module.load_extension = lambda: native
    cuda_module = importlib.import_module("nano_ep.backends.cuda")
    cuda_module.load_extension = lambda: native
    return importlib.import_module("nano_ep")


if __name__ == "__main__":
    module = build(verbose="--verbose" in sys.argv, skip_peer_device_checks="--skip-peer-device-checks" in sys.argv)
    print("built", module.__file__ if hasattr(module, "__file__") else BUILD_DIR / f"{NAME}.so")
