"""Compiles the CUDA sources of this folder for sm_100a, one shared library per source file.

A library is built the first time a kernel from it is asked for, with plain ``nvcc``
(no framework headers, so a file compiles in seconds), and is kept in ``_build/`` beside
the sources under a name that carries a hash of the source, the shared header and the
flags: an edited source is rebuilt, an unchanged one is loaded as it is.  A model
therefore compiles only what it uses.  While a build runs a line is printed now and then
to standard error.  If ``_build/`` cannot be written the build goes to
``$TESSERACT_B200_BUILD_DIR`` or a per-user folder under the system's temporary folder.
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
from typing import Dict, Iterable, List, Optional, Sequence

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "-Xcudafe", "--diag_suppress=177"]

# Files a source includes besides common.cuh and its own header (they count for its hash).
INCLUDES: Dict[str, List[str]] = {
    "attention_noalloc": ["attention_mma.cu", "attention_noalloc.h"],
    "attention_tcgen05": ["tma.cuh"],
    "gemm_tcgen05": ["tma.cuh", "umma.cuh"],
    "skinny_tcgen05": ["tma.cuh", "umma.cuh"],
}

# Every source file, with the extra flags it needs.
SOURCES: Dict[str, List[str]] = {
    "elementwise": [],
    "norm": [],
    "rope_cache": [],
    "attention_rows": [],
    "attention_mma": [],
    "attention_noalloc": [],
    "attention_tcgen05": [],
    "gemm_f32": [],
    "decode_linear": [],
    "gemm_tcgen05": [],
    "skinny_tcgen05": [],
    "sampling": [],
}


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels of tesseract_b200 cannot be built")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = tempfile.NamedTemporaryFile(dir=path, prefix=".probe", delete=True)
        probe.close()
        return True
    except OSError:
        return False


_build_dir_cache: Optional[str] = None


def build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache:
        return _build_dir_cache
    candidates = []
    if os.environ.get("TESSERACT_B200_BUILD_DIR"):
        candidates.append(os.environ["TESSERACT_B200_BUILD_DIR"])
    candidates.append(os.path.join(CSRC_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"tesseract_b200_build_{os.getuid()}"))
    for path in candidates:
        if _writable_dir(path):
            _build_dir_cache = path
            return path
    raise KernelBuildError(f"no writable build folder among {candidates}")


def _digest(name: str, flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for path in (os.path.join(CSRC_DIR, name + ".cu"), os.path.join(CSRC_DIR, "common.cuh")):
        with open(path, "rb") as handle:
            h.update(handle.read())
    for extra in [name + ".cuh"] + INCLUDES.get(name, []):
        extra = os.path.join(CSRC_DIR, extra)
        if os.path.exists(extra):
            with open(extra, "rb") as handle:
                h.update(handle.read())
    h.update(" ".join(list(ARCH_FLAGS) + list(BASE_FLAGS) + list(flags)).encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    flags = SOURCES[name]
    return os.path.join(build_dir(), f"libtb_{name}-{_digest(name, flags)}.so")


def _compile(name: str, out_path: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    tmp_path = f"{out_path}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *SOURCES[name], "-I", CSRC_DIR,
           os.path.join(CSRC_DIR, name + ".cu"), "-o", tmp_path]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    env = dict(os.environ)
    # nvcc writes temporaries under TMPDIR; an empty HOME is no obstacle.
    started = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)
    lines: List[str] = []

    def pump():
        for line in proc.stdout:
            lines.append(line)

    reader = threading.Thread(target=pump, daemon=True)
    reader.start()
    next_note = 10.0
    while proc.poll() is None:
        time.sleep(0.2)
        elapsed = time.time() - started
        if elapsed >= next_note:
            print(f"[tesseract_b200] still compiling {name}.cu for sm_100a ({elapsed:.0f} s)", file=sys.stderr,
                  flush=True)
            next_note += 10.0
    reader.join()
    output = "".join(lines)
    if proc.returncode != 0:
        try:
            os.unlink(tmp_path)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{output}")
    os.replace(tmp_path, out_path)
    prefix = f"libtb_{name}-"
    for stale in os.listdir(os.path.dirname(out_path)):       # older builds of this source are of no use
        if stale.startswith(prefix) and stale.endswith(".so") and stale != os.path.basename(out_path):
            try:
                os.unlink(os.path.join(os.path.dirname(out_path), stale))
            except OSError:
                pass
    if verbose and output:
        print(output, file=sys.stderr)


def ensure_built(names: Iterable[str], verbose: bool = False) -> Dict[str, str]:
    """Build (in parallel) whichever of ``names`` has no up-to-date library; return their paths."""
    names = list(dict.fromkeys(names))
    paths = {name: library_path(name) for name in names}
    todo = [name for name in names if not os.path.exists(paths[name])]
    if todo:
        print(f"[tesseract_b200] compiling CUDA kernels for sm_100a: {', '.join(todo)}", file=sys.stderr, flush=True)
        started = time.time()
        errors: List[BaseException] = []

        def work(name: str):
            try:
                _compile(name, paths[name], verbose)
            except BaseException as exc:  # noqa: BLE001 - reported below
                errors.append(exc)

        threads = [threading.Thread(target=work, args=(name,)) for name in todo]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        print(f"[tesseract_b200] compiled {len(todo)} kernel file(s) in {time.time() - started:.1f} s",
              file=sys.stderr, flush=True)
    return paths


_loaded: Dict[str, ctypes.CDLL] = {}
_load_lock = threading.Lock()


def load_library(name: str) -> ctypes.CDLL:
    """The shared library built from ``<name>.cu``, compiled first if needed."""
    with _load_lock:
        lib = _loaded.get(name)
        if lib is None:
            if name not in SOURCES:
                raise KernelBuildError(f"unknown kernel source '{name}'")
            path = ensure_built([name])[name]
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelBuildError(f"cannot load {path}: {exc}") from exc
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = False) -> Dict[str, str]:
    return ensure_built(SOURCES.keys(), verbose=verbose)


if __name__ == "__main__":
    for lib_name, lib_path in build_all(verbose="-v" in sys.argv).items():
        print(lib_name, lib_path)
