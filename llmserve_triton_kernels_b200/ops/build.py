"""Compiles the CUDA sources under ``csrc/`` into one shared library for sm_100a.

The kernels have a plain C interface, so they are compiled by nvcc alone (no Python or torch
headers: seconds per file) and loaded with ctypes.  The library lives beside this file; when the
package folder cannot be written, in a per-user folder under the system's temporary directory.
A build happens when the library is missing or older than a source, at the first kernel call or
through :func:`build`, and prints a line per file and a heartbeat while nvcc runs.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent.parent
CSRC = PACKAGE_DIR / "csrc"
LIB_NAME = "libllmserve_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# a profiling build whose decode kernels leave global-timer stamps per CTA (csrc/timeline.cuh); built into a folder of
# its own so that it never stands in for the product's library
def timeline_build() -> bool:
    return bool(os.environ.get("LLMSERVE_B200_TIMELINE"))


NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden"]


def _say(msg: str) -> None:
    print(f"[llmserve_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (
        os.environ.get("NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
    ):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise RuntimeError("nvcc was not found (looked at $NVCC, PATH and $CUDA_HOME/bin); the CUDA kernels cannot be built")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _writable(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dirs() -> tuple[Path, Path]:
    """``(folder of object files, folder of the library)``."""
    override = os.environ.get("LLMSERVE_B200_BUILD_DIR")
    if override:  # objects and library in a folder of the caller's choosing
        base = Path(override).resolve()
        return base / "obj", base
    lib_dir = PACKAGE_DIR / "ops"
    obj_dir = CSRC / "_build"
    if not timeline_build() and _writable(lib_dir) and _writable(obj_dir):
        return obj_dir, lib_dir
    tag = hashlib.sha1((str(PACKAGE_DIR) + ("+timeline" if timeline_build() else "")).encode()).hexdigest()[:12]
    base = Path(tempfile.gettempdir()) / f"llmserve_b200_{os.getuid()}_{tag}"
    base.mkdir(parents=True, exist_ok=True)
    return base / "obj", base


def library_path() -> Path:
    return build_dirs()[1] / LIB_NAME


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.is_file():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str], label: str) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"{label} failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if proc.stderr.strip() and os.environ.get("LLMSERVE_B200_VERBOSE_BUILD"):
        _say(proc.stderr.strip())


def build(force: bool = False, verbose_ptxas: bool = False) -> Path:
    """Compile what is out of date and link the library; returns its path."""
    obj_dir, lib_dir = build_dirs()
    obj_dir.mkdir(parents=True, exist_ok=True)
    lib = lib_dir / LIB_NAME
    srcs, hdrs = sources(), _headers()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    if not force and not _stale(lib, srcs + hdrs):
        return lib
    nvcc = find_nvcc()
    todo = [s for s in srcs if force or _stale(obj_dir / (s.stem + ".o"), [s] + hdrs)]
    _say(f"compiling {len(todo)} of {len(srcs)} CUDA files for sm_100a with {nvcc}")
    done = threading.Event()

    def heartbeat():
        start = time.time()
        while not done.wait(10.0):
            _say(f"still compiling ({time.time() - start:.0f} s)")

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    try:
        def compile_one(src: Path) -> None:
            obj = obj_dir / (src.stem + ".o")
            flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + (["-DLLM_TIMELINE"] if timeline_build() else [])
            _run([nvcc, *ARCH_FLAGS, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], f"nvcc {src.name}")
            _say(f"compiled {src.name}")

        with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as pool:
            list(pool.map(compile_one, todo))
        tmp = lib_dir / f".{LIB_NAME}.{os.getpid()}.tmp"
        objs = [str(obj_dir / (s.stem + ".o")) for s in srcs]
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *objs], "link")
        os.replace(tmp, lib)
    finally:
        done.set()
    _say(f"built {lib}")
    return lib
