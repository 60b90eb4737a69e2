"""Building and loading the CUDA libraries of `llm_b200/csrc`.

Every `.cu` file becomes one shared library, compiled for sm_100a with nvcc
the first time an operation from it is needed (the engine of MythEclipse/llm
compiles its one kernel file at build time instead, apps/engine/build.rs:66-72).
A library's file name carries a hash of its sources and flags, so a changed
source is rebuilt and an unchanged one is loaded as it is. Libraries are kept
in `llm_b200/csrc/_build/`; if that folder cannot be written, in a per-user
folder under the system's temporary directory.
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

from ..errors import KernelError

CSRC = Path(__file__).resolve().parent.parent / "csrc"
# no fast-math flag: expf, sqrtf and division keep their precise forms everywhere
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared"]

_loaded: dict = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


def _nvcc() -> str:
    for candidate in (os.environ.get("LLMB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise KernelError("nvcc was not found (looked at $LLMB_NVCC, PATH and /usr/local/cuda/bin); "
                      "the CUDA libraries of llm_b200 cannot be built")


def _headers() -> list:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _extra_flags() -> list:
    """More nvcc flags from $LLMB_NVCC_FLAGS (for instance -DLLMB_TRACE); they are part of a
    library's hash, so such a build lies beside the plain one."""
    return os.environ.get("LLMB_NVCC_FLAGS", "").split()


def _digest(source: Path) -> str:
    h = hashlib.sha256()
    for path in [source] + _headers():
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS + _extra_flags()).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> list:
    dirs = []
    if os.environ.get("LLMB_BUILD_DIR"):
        dirs.append(Path(os.environ["LLMB_BUILD_DIR"]))
    dirs.append(CSRC / "_build")
    dirs.append(Path(tempfile.gettempdir()) / f"llm_b200-build-{os.getuid()}")
    return dirs


_chosen_dir = None


def _writable_dir() -> Path:
    """The first build folder that can be written, found once per process."""
    global _chosen_dir
    with _dir_lock:
        if _chosen_dir is not None:
            return _chosen_dir
        for d in _build_dirs():
            try:
                d.mkdir(parents=True, exist_ok=True)
                probe = d / f".probe-{os.getpid()}-{threading.get_ident()}"
                probe.write_bytes(b"")
                probe.unlink()
                _chosen_dir = d
                return d
            except OSError:
                continue
    raise KernelError("no writable folder for the compiled CUDA libraries")


def library_path(name: str) -> Path | None:
    """The built library of csrc/<name>.cu if it exists already."""
    file_name = f"llmb_{name}-{_digest(CSRC / (name + '.cu'))}.so"
    for d in _build_dirs():
        if (d / file_name).is_file():
            return d / file_name
    return None


def _say(text: str) -> None:
    print(f"[llm_b200] {text}", file=sys.stderr, flush=True)


def compile_library(name: str) -> Path:
    source = CSRC / (name + ".cu")
    if not source.is_file():
        raise KernelError(f"no kernel source {source}")
    existing = library_path(name)
    if existing is not None:
        return existing
    out_dir = _writable_dir()
    target = out_dir / f"llmb_{name}-{_digest(source)}.so"
    scratch = out_dir / f".{target.name}.{os.getpid()}.{threading.get_ident()}.tmp"
    command = [_nvcc(), *NVCC_FLAGS, *_extra_flags(), "-I", str(CSRC), "-o", str(scratch), str(source), "-lcuda"]
    started = time.time()
    _say(f"compiling {source.name} for sm_100a ...")
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                               cwd=str(out_dir))
    while True:
        try:
            output, _ = process.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {source.name} ({time.time() - started:.0f} s)")
    if process.returncode != 0:
        try:
            scratch.unlink()
        except OSError:
            pass
        raise KernelError(f"nvcc failed on {source.name}:\n{output}")
    os.replace(scratch, target)
    for stale in ([] if _extra_flags() else out_dir.glob(f"llmb_{name}-*.so")):      # earlier builds of this source
        if stale != target:
            try:
                stale.unlink()
            except OSError:
                pass
    _say(f"built {target.name} in {time.time() - started:.1f} s")
    return target


def ensure_built(names) -> None:
    """Compile, in parallel, every library of `names` that is not built yet."""
    todo = [n for n in dict.fromkeys(names) if n not in _loaded and library_path(n) is None]
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 2)) as pool:
        list(pool.map(compile_library, todo))


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library of csrc/<name>.cu, compiled first if need be. Fails
    with KernelError (never falls back to another implementation)."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        path = compile_library(name)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelError(f"cannot load {path}: {error}") from None
        _loaded[name] = lib
        return lib


def all_sources() -> list:
    return sorted(p.stem for p in CSRC.glob("*.cu"))


_nvcc_version = None


def nvcc_version() -> str:
    """'12.9.86' from `nvcc --version` ('unknown' if nvcc cannot be run)."""
    global _nvcc_version
    if _nvcc_version is None:
        try:
            text = subprocess.run([_nvcc(), "--version"], capture_output=True, text=True, timeout=30).stdout
            _nvcc_version = text.rsplit("V", 1)[1].split()[0] if "V" in text else "unknown"
        except (KernelError, OSError, subprocess.SubprocessError, IndexError):
            _nvcc_version = "unknown"
    return _nvcc_version


def build_identity() -> str:
    """One hash over every kernel source, the host library's sources, the compiler flags and the
    compiler's version: two runs with equal identities ran the same native code (the build
    manifest of MythEclipse/llm records the same things, apps/engine/build.rs:30-62 and
    manifest.rs)."""
    h = hashlib.sha256()
    for name in all_sources():
        h.update(f"{name}:{_digest(CSRC / (name + '.cu'))};".encode())
    h.update(f"host:{_host_digest()};nvcc:{nvcc_version()}".encode())
    return h.hexdigest()[:16]


# ----------------------------------------------------------------------------- the host library

HOST = CSRC / "host"
# -ffp-contract=off: the random-weights generator must round every operation as the device does
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-ffp-contract=off", "-pthread"]
_host_lib = None


def _host_compiler() -> list:
    for candidate in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if candidate and (Path(candidate).is_file() or shutil.which(candidate)):
            return [candidate, *HOST_FLAGS]
    # nvcc drives a host compiler of its own choice
    return [_nvcc(), "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
            "-Xcompiler", "-ffp-contract=off", "-Xcompiler", "-pthread"]


def _host_digest() -> str:
    h = hashlib.sha256()
    for path in sorted(HOST.glob("*.cpp")) + sorted(HOST.glob("*.hpp")) + [CSRC / "plan.h", CSRC / "random_normal.h"]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()[:16]


def host_library_path() -> Path | None:
    file_name = f"llmb_host-{_host_digest()}.so"
    for d in _build_dirs():
        if (d / file_name).is_file():
            return d / file_name
    return None


def compile_host_library() -> Path:
    """csrc/host/*.cpp as one shared library (no CUDA in it): the cache's bookkeeping, the step
    packer, the scratch planner and the safetensors reader."""
    existing = host_library_path()
    if existing is not None:
        return existing
    out_dir = _writable_dir()
    target = out_dir / f"llmb_host-{_host_digest()}.so"
    scratch = out_dir / f".{target.name}.{os.getpid()}.{threading.get_ident()}.tmp"
    sources = [str(p) for p in sorted(HOST.glob("*.cpp"))]
    started = time.time()
    _say("compiling the host library ...")
    process = subprocess.run([*_host_compiler(), "-o", str(scratch), *sources], stdout=subprocess.PIPE,
                             stderr=subprocess.STDOUT, text=True, cwd=str(out_dir))
    if process.returncode != 0:
        try:
            scratch.unlink()
        except OSError:
            pass
        raise KernelError(f"the host library failed to compile:\n{process.stdout}")
    os.replace(scratch, target)
    for stale in out_dir.glob("llmb_host-*.so"):
        if stale != target:
            try:
                stale.unlink()
            except OSError:
                pass
    _say(f"built {target.name} in {time.time() - started:.1f} s")
    return target


def load_host_library() -> ctypes.CDLL:
    global _host_lib
    with _lock:
        if _host_lib is None:
            path = compile_host_library()
            try:
                _host_lib = ctypes.CDLL(str(path))
            except OSError as error:
                raise KernelError(f"cannot load {path}: {error}") from None
        return _host_lib
