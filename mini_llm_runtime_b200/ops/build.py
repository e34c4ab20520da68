"""Compiles the CUDA sources under ``csrc/`` for sm_100a, one shared library per ``.cu`` file,
and loads them with ``ctypes``.

The kernels expose plain ``extern "C"`` entry points that take device pointers and a stream, so
no Python or torch headers are involved and a file compiles in seconds.  A library is compiled
the first time it is asked for (only what the running model needs), into ``csrc/_build/`` next
to the sources when that folder can be written, else into a per-user folder under the system's
temporary directory.  The file name carries a hash of the source, the shared header and the
flags, so a stale library is never loaded.  Progress lines go to stderr while nvcc runs.

The reference builds its extension with ``torch.utils.cpp_extension.load`` and no architecture
flag (src/mini_llm_runtime/cuda_extension.py:11-35); here the target is always sm_100a.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
COMMON_FLAGS = ("-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden")

# name -> extra nvcc flags
LIBRARIES: dict[str, tuple[str, ...]] = {
    "elementwise": (),
    "linear_simt": (),
    "attention_generic": (),
    "sampling": (),
    "gemm_tcgen05": (),
    "attention_decode": (),
    "attention_mma": (),
    "gemm_skinny": (),
    "attention_tcgen05": (),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def register_library(name: str, flags: tuple[str, ...] = ()) -> None:
    LIBRARIES[name] = tuple(flags)


def _say(message: str) -> None:
    print(f"[mini_llm_runtime_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("MLR_NVCC"), shutil.which("nvcc")]
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            candidates.append(os.path.join(root, "bin", "nvcc"))
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise BuildError("nvcc was not found (looked at $MLR_NVCC, PATH, $CUDA_HOME, /usr/local/cuda); "
                     "the CUDA kernels cannot be built and there is no other backend")


def build_directory() -> Path:
    override = os.environ.get("MLR_BUILD_DIR")
    if override:
        path = Path(override)
        path.mkdir(parents=True, exist_ok=True)
        return path
    in_tree = CSRC / "_build"
    try:
        in_tree.mkdir(parents=True, exist_ok=True)
        probe = in_tree / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return in_tree
    except OSError:
        pass
    fallback = Path(tempfile.gettempdir()) / f"mini_llm_runtime_b200-build-{os.getuid()}"
    fallback.mkdir(parents=True, exist_ok=True)
    return fallback


def _source_hash(name: str, flags: tuple[str, ...]) -> str:
    digest = hashlib.sha256()
    digest.update((CSRC / f"{name}.cu").read_bytes())
    for header in sorted([*CSRC.glob("*.cuh"), *CSRC.glob("*.h")]):
        digest.update(header.name.encode())
        digest.update(header.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + flags).encode())
    return digest.hexdigest()[:16]


def library_path(name: str, directory: Path | None = None) -> Path:
    flags = LIBRARIES[name]
    directory = directory or build_directory()
    return directory / f"mlr_{name}-{_source_hash(name, flags)}.so"


def _find_built(name: str) -> Path | None:
    """A current library in the in-tree folder (it may be read-only) or in the writable one."""
    flags = LIBRARIES[name]
    file_name = f"mlr_{name}-{_source_hash(name, flags)}.so"
    for directory in (CSRC / "_build", build_directory()):
        candidate = directory / file_name
        if candidate.is_file():
            return candidate
    return None


def _run_nvcc(command: list[str], label: str) -> None:
    started = time.monotonic()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker() -> None:
        while not done.wait(10.0):
            _say(f"still compiling {label} ({time.monotonic() - started:.0f} s)")

    thread = threading.Thread(target=ticker, daemon=True)
    thread.start()
    try:
        output, _ = process.communicate()
    finally:
        done.set()
    if process.returncode != 0:
        raise BuildError(f"nvcc failed on {label} (exit {process.returncode}):\n{output}")
    _say(f"compiled {label} in {time.monotonic() - started:.1f} s")


def compile_library(name: str, *, verbose_ptxas: bool = False) -> Path:
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library {name!r}; known: {', '.join(sorted(LIBRARIES))}")
    built = _find_built(name)
    if built is not None and not verbose_ptxas:
        return built
    directory = build_directory()
    target = library_path(name, directory)
    nvcc = find_nvcc()
    lock_path = directory / f".{name}.lock"
    with open(lock_path, "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        try:
            if target.is_file() and not verbose_ptxas:
                return target
            scratch = directory / f".{target.name}.{os.getpid()}.tmp"
            command = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *LIBRARIES[name], "-I", str(CSRC),
                       "-o", str(scratch), str(CSRC / f"{name}.cu")]
            if verbose_ptxas:
                command[1:1] = ["-Xptxas", "-v"]
            _say(f"compiling {name}.cu for sm_100a (first use; kept in {directory})")
            try:
                _run_nvcc(command, f"{name}.cu")
                os.replace(scratch, target)
            finally:
                if scratch.exists():
                    scratch.unlink()
            for stale in directory.glob(f"mlr_{name}-*.so"):
                if stale != target:
                    try:
                        stale.unlink()
                    except OSError:
                        pass
        finally:
            fcntl.flock(lock_file, fcntl.LOCK_UN)
    return target


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library ``name``; compiled first if no current build exists."""
    with _lock:
        if name not in _loaded:
            path = compile_library(name)
            try:
                _loaded[name] = ctypes.CDLL(str(path))
            except OSError as error:
                raise BuildError(f"cannot load {path}: {error}") from error
            if hasattr(_loaded[name], "mlr_set_pdl"):
                _loaded[name].mlr_set_pdl(int(_pdl))
        return _loaded[name]


_pdl = os.environ.get("MLR_PDL", "1") != "0"


def set_programmatic_launch(enabled: bool) -> None:
    """Launch kernels so that each may start while its predecessor on the stream still runs
    (programmatic dependent launch).  On by default; MLR_PDL=0 in the environment turns it off."""
    global _pdl
    _pdl = bool(enabled)
    with _lock:
        for library in _loaded.values():
            if hasattr(library, "mlr_set_pdl"):
                library.mlr_set_pdl(int(_pdl))


def build_all() -> dict[str, Path]:
    return {name: compile_library(name) for name in LIBRARIES}
