"""Compiles the CUDA sources under ``csrc/`` for sm_100a and loads them.

The kernels are plain CUDA with ``extern "C"`` launchers on raw pointers, so
they compile in seconds with nvcc alone (no torch headers) and are loaded with
ctypes.  A library is compiled at its first use and kept beside the sources
(``csrc/_build/``), or in a per-user temporary folder when the package folder
is not writable; its file name carries a hash of the sources and flags, so an
edited source is recompiled and a stale library is never loaded.

There is no fallback: if nvcc is missing or a compile fails, ``KernelBuildError``
says so and nothing runs.
"""

from __future__ import annotations

import ctypes
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def _log(msg: str) -> None:
    print(f"[simple_inference_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError(
        "nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels "
        "cannot be compiled and there is no other path"
    )


def build_dir() -> Path:
    """In-tree when writable, else a per-user folder under the temp dir."""
    cand = CSRC / "_build"
    try:
        cand.mkdir(exist_ok=True)
        probe = cand / f".w{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return cand
    except OSError:
        alt = Path(tempfile.gettempdir()) / f"simple_inference_b200_build_{os.getuid()}"
        alt.mkdir(parents=True, exist_ok=True)
        return alt


def _digest(sources: list[Path], defines: list[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sources:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + defines).encode())
    return h.hexdigest()[:16]


def _run(cmd: list[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker() -> None:
        while not done.wait(10.0):
            _log(f"still compiling {what} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {what}:\n{' '.join(cmd)}\n{out}")


def library_path(name: str, source_names: list[str], defines: list[str] | None = None) -> Path:
    """Build (if needed) and return the shared library made from ``source_names``."""
    defines = list(defines or [])
    sources = [CSRC / s for s in source_names]
    for s in sources:
        if not s.is_file():
            raise KernelBuildError(f"kernel source {s} is missing")
    out = build_dir() / f"lib{name}_{_digest(sources, defines)}.so"
    if out.is_file():
        return out
    nvcc = _nvcc()
    _log(f"compiling {name} for sm_100a ({', '.join(source_names)}) -> {out}")
    t0 = time.time()
    with tempfile.TemporaryDirectory(prefix="si_b200_obj_") as tmp:
        objs = [Path(tmp) / (s.stem + ".o") for s in sources]

        def compile_one(pair: tuple[Path, Path]) -> None:
            src, obj = pair
            _run([nvcc, *NVCC_FLAGS, *defines, "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
                 src.name)

        with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 4)) as pool:
            list(pool.map(compile_one, zip(sources, objs)))
        tmp_out = out.with_suffix(f".tmp{os.getpid()}")
        _run([nvcc, "-shared", "-o", str(tmp_out), *[str(o) for o in objs]], f"link {name}")
        os.replace(tmp_out, out)
    _log(f"built {out.name} in {time.time() - t0:.1f} s")
    return out


def load_library(name: str, source_names: list[str], defines: list[str] | None = None) -> ctypes.CDLL:
    key = name + "|" + " ".join(defines or [])
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(str(library_path(name, source_names, defines)))
            _loaded[key] = lib
        return lib
