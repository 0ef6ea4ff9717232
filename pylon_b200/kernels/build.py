"""Builds the CUDA sources under ``pylon_b200/csrc`` for sm_100a and loads them.

Each ``.cu`` file becomes one shared library with a C interface, built with ``nvcc`` the
first time something needs it and reused afterwards (a stamp of the sources and flags
decides).  Libraries are written next to the sources (``csrc/_build``) when that folder
can be written, else under ``$PYLON_B200_BUILD_DIR`` or the system's temporary folder, so
a read-only checkout or a user without a home directory still works.  While the compiler
runs, a line is printed to stderr now and then.

There is no fallback: a missing compiler or a failed build raises :class:`KernelBuildError`.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Iterable, Optional

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
COMMON_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr")


class KernelBuildError(RuntimeError):
    pass


_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _say(text: str) -> None:
    print(f"[pylon_b200] {text}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (
        os.environ.get("PYLON_B200_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise KernelBuildError("nvcc was not found (looked at $PYLON_B200_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin)")


def build_dir() -> Path:
    """The folder libraries are written to: the first of the candidates that can be written."""
    candidates = []
    if os.environ.get("PYLON_B200_BUILD_DIR"):
        candidates.append(Path(os.environ["PYLON_B200_BUILD_DIR"]))
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"pylon_b200_build_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for built kernels among {[str(c) for c in candidates]}")


def _stamp(sources: Iterable[Path], flags: Iterable[str]) -> str:
    digest = hashlib.sha256()
    for path in sorted(set(sources)):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update("\0".join(flags).encode())
    return digest.hexdigest()[:16]


def library_name(source: str, defines: Optional[dict[str, int]] = None) -> str:
    stem = Path(source).stem
    if defines:
        stem += "".join(f"_{key.lower()}{value}" for key, value in sorted(defines.items()))
    return f"libpylon_{stem}.so"


def _compile(source: Path, target: Path, flags: list[str]) -> None:
    nvcc = find_nvcc()
    temporary = target.with_suffix(f".tmp{os.getpid()}.so")
    command = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *flags, "-I", str(CSRC), "-o", str(temporary), str(source)]
    _say(f"compiling {source.name} for sm_100a -> {target.name}")
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    output: list[str] = []
    reader = threading.Thread(target=lambda: output.append(process.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            process.wait(timeout=10)
            break
        except subprocess.TimeoutExpired:
            _say(f"  still compiling {source.name} ({time.time() - started:.0f} s)")
    reader.join()
    if process.returncode != 0:
        temporary.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed on {source.name} (exit {process.returncode}):\n{''.join(output)}")
    os.replace(temporary, target)
    _say(f"  built {target.name} in {time.time() - started:.1f} s")


def load(source: str, defines: Optional[dict[str, int]] = None, extra_flags: Iterable[str] = ()) -> ctypes.CDLL:
    """Build (if needed) and load the library of ``csrc/<source>``.

    ``defines`` become ``-D`` options and part of the library's name, so that one source
    can be built for several compile-time sizes.
    """
    name = library_name(source, defines)
    with _lock:
        if name in _loaded:
            return _loaded[name]
        path = CSRC / source
        if not path.is_file():
            raise KernelBuildError(f"kernel source {path} is missing")
        flags = [f"-D{key}={value}" for key, value in sorted((defines or {}).items())] + list(extra_flags)
        headers = list(CSRC.glob("*.cuh"))
        stamp = _stamp([path, *headers], [*ARCH_FLAGS, *COMMON_FLAGS, *flags])
        folder = build_dir()
        target = folder / name
        stamp_file = folder / (name + ".stamp")
        lock_file = folder / (name + ".lock")
        with open(lock_file, "w") as handle:
            fcntl.flock(handle, fcntl.LOCK_EX)
            try:
                current = stamp_file.read_text().strip() if stamp_file.is_file() else ""
                if not target.is_file() or current != stamp:
                    _compile(path, target, flags)
                    stamp_file.write_text(stamp)
            finally:
                fcntl.flock(handle, fcntl.LOCK_UN)
        try:
            library = ctypes.CDLL(str(target))
        except OSError as error:
            raise KernelBuildError(f"could not load {target}: {error}") from error
        library.pylon_last_error.restype = ctypes.c_char_p
        _loaded[name] = library
        return library


def build_all() -> list[str]:
    """Compile every library the engine can use with its default sizes; returns their names."""
    from pylon_b200.kernels import ops

    return ops.build_all()
