"""Builds the CUDA sources of ``csrc/`` into shared libraries with nvcc, for
sm_100a only, at the first call that needs them.

Each library is one ``.cu`` file (plus the headers beside it) and is named by
a hash of its sources and flags, so an edited source is rebuilt and an
unchanged one is found again.  Libraries are written beside the sources (in
``csrc/_build``) when that folder can be written, else into a per-user folder
under the system's temporary directory.  While nvcc runs, a line is printed
every few seconds, since a first call in a fresh checkout can take a minute.

The reference builds with a Makefile for sm_86/sm_61 (Makefile:5,177-180) and
loads ``build/libmini_llm_gpu.so`` through ctypes
(pytorch/src/mini_llm/native.py:203-214); the binding manner is kept, the
build happens on demand.
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

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
]

# library name -> source file.  Headers (*.cuh) beside them enter every hash.
LIBRARIES = {
    "plain": "plain_kernels.cu",
    "sampling": "sampling_kernels.cu",
    "decode": "decode_kernels.cu",
    "gemm": "gemm_tcgen05.cu",
    "attention": "attention_tcgen05.cu",
    "fused": "fused_decode.cu",
}

_lock = threading.Lock()
_built: dict[str, str] = {}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    candidates = []
    for env in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(env):
            candidates.append(os.path.join(os.environ[env], "bin", "nvcc"))
    on_path = shutil.which("nvcc")
    if on_path:
        candidates.append(on_path)
    candidates.append("/usr/local/cuda/bin/nvcc")
    for path in candidates:
        if os.path.isfile(path) and os.access(path, os.X_OK):
            return path
    raise BuildError("nvcc was not found (looked at $CUDA_HOME, $PATH and /usr/local/cuda); "
                     "the CUDA kernels cannot be built and there is no fallback path")


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cuh") or f.endswith(".h"))


def _source_hash(source: str, extra_flags=()) -> str:
    digest = hashlib.sha256()
    for name in [source, *_headers()]:
        with open(os.path.join(CSRC, name), "rb") as handle:
            digest.update(name.encode())
            digest.update(handle.read())
    digest.update(" ".join([*NVCC_FLAGS, *extra_flags]).encode())
    return digest.hexdigest()[:16]


def _build_dirs() -> list[str]:
    dirs = [os.path.join(CSRC, "_build")]
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(os.path.join(tempfile.gettempdir(), f"mini_llm_b200-build-{uid}"))
    return dirs


def _writable_dir() -> str:
    for path in _build_dirs():
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe-{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError("no folder to build the CUDA kernels in: tried " + ", ".join(_build_dirs()))


def library_path(name: str, build: bool = True) -> str:
    """Path of the built library ``name``; builds it first if it is missing."""
    with _lock:
        if name in _built:
            return _built[name]
        if name not in LIBRARIES:
            raise BuildError(f"unknown kernel library '{name}'")
        source = LIBRARIES[name]
        file_name = f"libmllm_{name}-{_source_hash(source)}.so"
        for folder in _build_dirs():
            path = os.path.join(folder, file_name)
            if os.path.isfile(path):
                _built[name] = path
                return path
        if not build:
            raise BuildError(f"kernel library '{name}' is not built")
        path = os.path.join(_writable_dir(), file_name)
        _compile(os.path.join(CSRC, source), path, name)
        _built[name] = path
        return path


def _compile(source: str, target: str, name: str) -> None:
    nvcc = find_nvcc()
    partial = f"{target}.{os.getpid()}.tmp"
    command = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-o", partial, source]
    started = time.time()
    print(f"[mini_llm_b200] compiling {os.path.basename(source)} for sm_100a ...", file=sys.stderr, flush=True)
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    output = []
    reader = threading.Thread(target=lambda: output.append(process.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            process.wait(timeout=10)
            break
        except subprocess.TimeoutExpired:
            print(f"[mini_llm_b200] still compiling {name} ({time.time() - started:.0f} s)",
                  file=sys.stderr, flush=True)
    reader.join()
    if process.returncode != 0:
        if os.path.exists(partial):
            os.remove(partial)
        raise BuildError(f"nvcc failed on {source}:\n{''.join(output)}")
    os.replace(partial, target)      # atomic: a concurrent process never sees half a file
    _drop_older_builds(target, name)
    print(f"[mini_llm_b200] built {os.path.basename(target)} in {time.time() - started:.0f} s",
          file=sys.stderr, flush=True)


def _drop_older_builds(target: str, name: str) -> None:
    """Builds of earlier versions of the same source (other hashes) in the folder of a fresh
    build are of no use any more.  A process that still has one mapped keeps its mapping."""
    folder, keep = os.path.dirname(target), os.path.basename(target)
    prefix = f"libmllm_{name}-"
    for entry in os.listdir(folder):
        if entry.startswith(prefix) and entry.endswith(".so") and entry != keep:
            try:
                os.remove(os.path.join(folder, entry))
            except OSError:
                pass


def build_all() -> dict[str, str]:
    """Build every library (in parallel); returns name -> path."""
    errors = []
    threads = []
    # library_path holds a lock while it compiles, so the missing libraries are
    # found first and then compiled side by side, one nvcc process each.
    missing = []
    for lib, source in LIBRARIES.items():
        try:
            library_path(lib, build=False)
        except BuildError:
            missing.append(lib)
    if missing:
        folder = _writable_dir()
        for lib in missing:
            source = LIBRARIES[lib]
            target = os.path.join(folder, f"libmllm_{lib}-{_source_hash(source)}.so")
            thread = threading.Thread(target=lambda s=source, t=target, n=lib: _guarded(s, t, n, errors))
            thread.start()
            threads.append(thread)
        for thread in threads:
            thread.join()
    if errors:
        raise errors[0]
    return {lib: library_path(lib) for lib in LIBRARIES}


def _guarded(source, target, name, errors):
    try:
        _compile(os.path.join(CSRC, source), target, name)
    except Exception as error:
        errors.append(error)
