"""Builds and loads the CUDA libraries of ``tinyinfer_b200/csrc`` (sm_100a only).

Each library is a plain shared object with ``extern "C"`` launchers, compiled by ``nvcc`` at its
first use and kept in ``tinyinfer_b200/csrc/_build`` (or, if the checkout is read-only, in a
per-user folder under the system's temporary directory). The file name carries a hash of the
sources and flags, so an edited kernel is rebuilt and a stale object is never loaded. A library
is only built when something asks for it: a 32-bit run never compiles the tensor-core kernels.

There is no fallback: if ``nvcc`` or the build fails, loading raises.
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
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, List

CSRC = Path(__file__).resolve().parent.parent / "csrc"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler",
                "-fvisibility=hidden"]

LIBRARIES: Dict[str, dict] = {
    # every dtype, every shape: the 32-bit path and the general bfloat16 path
    "core": dict(sources=["runtime.cu", "elementwise.cu", "rope_append.cu",
                          "attention_generic.cu", "gemm_simt.cu", "sampling.cu"],
                 headers=["common.cuh"], link=[]),
    # bfloat16 tensor-core kernels (tcgen05 + TMA); only a bfloat16 model loads it
    "sm100": dict(sources=["runtime.cu", "sm100_host.cu", "gemm_tcgen05.cu", "attention_mma.cu",
                           "attention_prefill_tcgen05.cu", "attention_prefill_pair_tcgen05.cu", "gemm_pair_tcgen05.cu"],
                  headers=["common.cuh", "sm100_ptx.cuh"], link=[]),
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def nvcc_path() -> str:
    for cand in (os.environ.get("TINYINFER_B200_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of tinyinfer_b200 cannot be built "
                     "(set TINYINFER_B200_NVCC or CUDA_HOME)")


def build_dir() -> Path:
    override = os.environ.get("TINYINFER_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates += [CSRC / "_build",
                   Path(tempfile.gettempdir()) / f"tinyinfer_b200-build-{os.getuid()}"]
    for cand in candidates:
        try:
            cand.mkdir(parents=True, exist_ok=True)
            probe = cand / f".probe-{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return cand
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(c) for c in candidates]}")


def _signature(name: str) -> str:
    spec = LIBRARIES[name]
    h = hashlib.sha1()
    for rel in list(spec["sources"]) + list(spec["headers"]):
        h.update(rel.encode())
        h.update((CSRC / rel).read_bytes())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + spec.get("flags", []) + spec["link"]).encode())
    return h.hexdigest()[:12]


def library_path(name: str) -> Path:
    return build_dir() / f"libti_{name}-{_signature(name)}.so"


def _say(msg: str) -> None:
    print(f"[tinyinfer_b200] {msg}", file=sys.stderr, flush=True)


def build(name: str, verbose: bool = True) -> Path:
    """Compiles library ``name`` if its current build is missing; returns the .so path."""
    if name not in LIBRARIES:
        raise KeyError(f"unknown library {name!r}; known: {sorted(LIBRARIES)}")
    out = library_path(name)
    if out.is_file():
        return out
    spec = LIBRARIES[name]
    nvcc = nvcc_path()
    folder = out.parent
    with open(folder / f".lock-{name}", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)           # another process may be building the same file
        if out.is_file():
            return out
        work = Path(tempfile.mkdtemp(prefix=f"obj-{name}-", dir=folder))
        sources: List[str] = spec["sources"]
        t0 = time.time()
        done = []
        stop = threading.Event()

        def ticker():
            while not stop.wait(10.0):
                _say(f"compiling {name}: {len(done)}/{len(sources)} files done, "
                     f"{time.time() - t0:.0f} s")

        def compile_one(rel: str) -> str:
            obj = work / (Path(rel).stem + ".o")
            cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *spec.get("flags", []), "-I", str(CSRC),
                   "-c", str(CSRC / rel), "-o", str(obj)]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise BuildError(f"nvcc failed on {rel}:\n{res.stdout}\n{res.stderr}")
            done.append(rel)
            return str(obj)

        if verbose:
            _say(f"compiling CUDA library '{name}' for sm_100a ({len(sources)} files) into {folder}")
        thread = threading.Thread(target=ticker, daemon=True)
        if verbose:
            thread.start()
        try:
            with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 2)) as pool:
                objects = list(pool.map(compile_one, sources))
            tmp = work / "lib.so"
            cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *objects, *spec["link"]]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise BuildError(f"link of {name} failed:\n{res.stdout}\n{res.stderr}")
            os.replace(tmp, out)
            for old in folder.glob(f"libti_{name}-*.so"):     # builds of earlier states of the sources
                if old != out:
                    try:
                        old.unlink()       # a process that has one loaded keeps its mapping
                    except OSError:
                        pass
        finally:
            stop.set()
            shutil.rmtree(work, ignore_errors=True)
        if verbose:
            _say(f"built {out.name} in {time.time() - t0:.0f} s")
    return out


def load(name: str) -> ctypes.CDLL:
    """The loaded library, built first if need be. Raises if that is impossible."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build(name)
            lib = ctypes.CDLL(str(path))
            lib.ti_last_error.restype = ctypes.c_char_p
            lib.ti_launch_count.restype = ctypes.c_longlong
            _loaded[name] = lib
        return lib


def loaded_libraries() -> Dict[str, ctypes.CDLL]:
    return dict(_loaded)


_replayed_launches = 0


def count_replayed_launches(n: int) -> None:
    """Kernels that ran as part of a replayed CUDA graph (they do not pass through the launchers)."""
    global _replayed_launches
    _replayed_launches += int(n)


def launch_count() -> int:
    """Kernels of this package launched by this process so far, directly or in a replayed graph."""
    return sum(int(lib.ti_launch_count()) for lib in _loaded.values()) + _replayed_launches


def build_all(verbose: bool = True) -> List[Path]:
    return [build(name, verbose) for name in LIBRARIES]
