"""Compiles the CUDA sources under `csrc/` for sm_100a and loads them with ctypes.

The kernels are plain `extern "C"` launchers that take raw device pointers and
a stream, so no torch header is compiled and a cold build takes seconds per
file. Objects are cached by a hash of source + headers + flags; the shared
objects live in-tree (`rllm_b200/_lib/`) when that is writable, else under the
system temp folder. Nothing here falls back to another backend: a missing
compiler or a failed build raises.
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

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")

# library name -> sources. "simt" holds the generic kernels of both precisions;
# "sm100" the tcgen05/TMA kernels that only the bfloat16 path calls; "host" the native
# bookkeeping of the cache manager (plain C++, no device code).
LIBRARIES: dict[str, list[str]] = {
    "simt": ["simt_basic.cu", "simt_gemm.cu", "simt_attention.cu", "sampling.cu"],
    "sm100": ["tc_gemm.cu", "stream_gemm.cu", "attn_fa.cu", "attn_decode.cu", "attn_prefill_tc.cu", "wait_probe.cu"],
    "host": ["host_runtime.cpp"],          # no CUDA: the cache manager's bookkeeping and metadata writer
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (set NVCC or put it on PATH); the CUDA kernels are "
                     "required and there is no fallback")


def _lib_dir() -> str:
    cand = os.environ.get("RLLM_B200_LIB_DIR") or os.path.join(os.path.dirname(_HERE), "_lib")
    try:
        os.makedirs(cand, exist_ok=True)
        probe = os.path.join(cand, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return cand
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"rllm_b200_lib_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(paths: list[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(os.path.join(CSRC, p), "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def _say(msg: str) -> None:
    print(f"[rllm_b200 build] {msg}", file=sys.stderr, flush=True)


def _run_with_heartbeat(cmd: list[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def beat():
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f}s)")

    th = threading.Thread(target=beat, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{out}")
    if os.environ.get("RLLM_B200_BUILD_VERBOSE") and out.strip():
        _say(out.strip())


def build_library(name: str, verbose_ptxas: bool = False) -> str:
    """Compile (if stale) and return the path of lib `name`."""
    srcs = [s for s in LIBRARIES[name] if os.path.isfile(os.path.join(CSRC, s))]
    if not srcs:
        raise BuildError(f"library {name!r} has no sources under {CSRC}")
    nvcc = _nvcc()
    # RLLM_B200_NVCC_FLAGS: extra compiler flags (e.g. -DNAME=value to try a tuning constant)
    flags = list(NVCC_FLAGS) + os.environ.get("RLLM_B200_NVCC_FLAGS", "").split() + \
        (["-Xptxas", "-v"] if verbose_ptxas else [])
    libdir = _lib_dir()
    hdrs = _headers()
    objs, jobs = [], []
    for s in srcs:
        tag = _digest([s] + hdrs, " ".join(flags))
        obj = os.path.join(libdir, f"{os.path.splitext(s)[0]}.{tag}.o")
        objs.append(obj)
        if not os.path.isfile(obj):
            jobs.append((s, obj))
    so_tag = hashlib.sha256(" ".join(os.path.basename(o) for o in objs).encode()).hexdigest()[:12]   # not the folder: a copied tree keeps its library
    so = os.path.join(libdir, f"librllm_b200_{name}.{so_tag}.so")
    if os.path.isfile(so) and not jobs:
        return so
    if jobs:
        _say(f"compiling {len(jobs)} source file(s) of '{name}' for sm_100a into {libdir} "
             f"(first use only)")

        def one(job):
            s, obj = job
            tmp = obj + f".tmp{os.getpid()}"
            _run_with_heartbeat([nvcc, *flags, "-I", CSRC, "-c", os.path.join(CSRC, s), "-o", tmp],
                                f"nvcc {s}")
            os.replace(tmp, obj)
            _say(f"compiled {s}")

        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(one, jobs))
    tmp = so + f".tmp{os.getpid()}"
    _run_with_heartbeat([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                         "-o", tmp, *objs, "-lcudart_static", "-ldl", "-lrt", "-lpthread"],
                        f"link {os.path.basename(so)}")
    os.replace(tmp, so)
    _say(f"built {os.path.basename(so)}")
    _prune(libdir, name, srcs, objs, so)
    return so


def _prune(libdir: str, name: str, srcs: list[str], objs: list[str], so: str) -> None:
    """Delete what earlier versions of the sources left behind (a loaded library stays mapped)."""
    keep = {os.path.basename(p) for p in objs} | {os.path.basename(so)}
    stems = tuple(os.path.splitext(s)[0] + "." for s in srcs)
    for f in os.listdir(libdir):
        stale_obj = f.endswith(".o") and f.startswith(stems)
        stale_so = f.endswith(".so") and f.startswith(f"librllm_b200_{name}.")
        if (stale_obj or stale_so) and f not in keep:
            try:
                os.remove(os.path.join(libdir, f))
            except OSError:
                pass


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library `name`, building it first when needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
        return lib


def build_all(verbose_ptxas: bool = False) -> dict[str, str]:
    return {name: build_library(name, verbose_ptxas) for name in LIBRARIES}
