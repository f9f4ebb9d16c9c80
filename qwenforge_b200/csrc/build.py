"""Builds and loads the CUDA kernel libraries.

Every `<name>.cu` beside this file is one shared library with a plain C interface
(`extern "C"` functions taking device pointers, sizes and a stream), compiled by nvcc for
sm_100a only and loaded with ctypes. A library is compiled the first time something asks
for it, so a run compiles what its model needs and nothing else; `build_all()` compiles
everything. A built file is named by a hash of its source, the shared headers and the
compiler flags, so an edited source is never served by a stale binary.

Built files go to `_build/` beside the sources when that folder can be written, else to
`$QWENFORGE_B200_BUILD_DIR`, else to a per-user folder under the system's temporary
directory. Nothing here needs HOME or a network.

There is no fallback: if nvcc is missing or a compilation fails, `KernelLibraryError`
says which file and why, and nothing runs.
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

_SRC = Path(__file__).resolve().parent
_NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]
_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelLibraryError(RuntimeError):
    pass


def library_names() -> list[str]:
    return sorted(p.stem for p in _SRC.glob("*.cu"))


def _say(message: str) -> None:
    print(f"[qwenforge_b200] {message}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    candidates = [os.environ.get("QWENFORGE_B200_NVCC"), shutil.which("nvcc")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            candidates.append(str(Path(home) / "bin" / "nvcc"))
    for c in candidates:
        if c and Path(c).exists():
            return c
    raise KernelLibraryError("nvcc not found (looked in PATH, $CUDA_HOME and /usr/local/cuda): the CUDA kernels of "
                             "this library cannot be built, and there is no other execution path")


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}-{threading.get_ident()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def _build_dir() -> Path:
    choices = [_SRC / "_build"]
    if os.environ.get("QWENFORGE_B200_BUILD_DIR"):
        choices.append(Path(os.environ["QWENFORGE_B200_BUILD_DIR"]))
    choices.append(Path(tempfile.gettempdir()) / f"qwenforge_b200-build-{os.getuid()}")
    for c in choices:
        if _writable(c):
            return c
    raise KernelLibraryError(f"no writable folder for built kernels (tried {', '.join(map(str, choices))})")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(_NVCC_FLAGS).encode())
    for path in sorted(_SRC.glob("*.cuh")) + sorted(_SRC.glob("*.h")) + [_SRC / f"{name}.cu"]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()[:16]


def _find_built(name: str, digest: str) -> Path | None:
    file_name = f"{name}.{digest}.so"
    places = [_SRC / "_build"]
    if os.environ.get("QWENFORGE_B200_BUILD_DIR"):
        places.append(Path(os.environ["QWENFORGE_B200_BUILD_DIR"]))
    places.append(Path(tempfile.gettempdir()) / f"qwenforge_b200-build-{os.getuid()}")
    for p in places:
        if (p / file_name).exists():
            return p / file_name
    return None


def _compile(name: str) -> Path:
    source = _SRC / f"{name}.cu"
    if not source.exists():
        raise KernelLibraryError(f"no kernel source {source.name}; known: {', '.join(library_names())}")
    digest = _digest(name)
    built = _find_built(name, digest)
    if built is not None:
        return built
    out_dir = _build_dir()
    target = out_dir / f"{name}.{digest}.so"
    partial = out_dir / f".{name}.{digest}.{os.getpid()}.{threading.get_ident()}.tmp.so"
    command = [_nvcc(), *_NVCC_FLAGS, "-I", str(_SRC), "-o", str(partial), str(source)]
    _say(f"compiling {source.name} for sm_100a ...")
    started = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", str(out_dir))
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    while True:
        try:
            output, _ = process.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {source.name} ({time.time() - started:.0f} s)")
    if process.returncode != 0:
        partial.unlink(missing_ok=True)
        raise KernelLibraryError(f"nvcc failed on {source.name} (exit {process.returncode}):\n{output}")
    os.replace(partial, target)
    for stale in out_dir.glob(f"{name}.*.so"):  # builds of earlier versions of this source
        if stale != target:
            stale.unlink(missing_ok=True)
    _say(f"compiled {source.name} in {time.time() - started:.1f} s")
    return target


def library(name: str) -> ctypes.CDLL:
    """The loaded library `name` (compiling it first if no current build exists)."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = _compile(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelLibraryError(f"cannot load {path}: {exc}") from exc
            _loaded[name] = lib
    return lib


def prepare(names) -> None:
    """Compile (in parallel) and load the named libraries; used when a model is built, so
    that all compilation happens up front with progress lines instead of inside the first step."""
    todo = [n for n in sorted(set(names)) if n not in _loaded]
    if not todo:
        return
    missing = [n for n in todo if _find_built(n, _digest(n)) is None]
    if missing:
        _say(f"{len(missing)} kernel librar{'y' if len(missing) == 1 else 'ies'} to compile: {', '.join(missing)}")
        with ThreadPoolExecutor(max_workers=min(8, len(missing))) as pool:
            list(pool.map(_compile, missing))
    for n in todo:
        library(n)


def build_all() -> list[str]:
    names = library_names()
    prepare(names)
    return names
