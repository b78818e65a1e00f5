"""Builds and loads the CUDA kernels of this package as one shared library.

The sources under ``sleuth_b200/csrc`` are compiled with ``nvcc`` for sm_100a into
``sleuth_b200/_build/libsleuth_b200.so`` (or, when the package folder cannot be written, into a
per-user folder under the system's temporary directory). The first call on a fresh checkout
compiles, printing a line per file; later calls load the finished library. A stamp file holding a
hash of the sources and flags decides whether the library is current.

There is no fallback: without ``nvcc`` or without a CUDA device the functions here raise.
The launchers are plain ``extern "C"`` functions taking device pointers as integers and the stream
as the last argument; they return 0 or a code whose message ``slb_last_error`` gives.
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
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]
# More flags for a build of one's own, e.g. SLEUTH_B200_NVCC_FLAGS=-DSLB_TIMELINE together with
# SLEUTH_B200_BUILD_DIR=<another folder> for a library whose kernels record a timeline (kernels/timeline.py).
NVCC_FLAGS += os.environ.get("SLEUTH_B200_NVCC_FLAGS", "").split()
LIB_NAME = "libsleuth_b200.so"

_lock = threading.Lock()
_lib = None


class KernelBuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[sleuth_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("SLEUTH_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise KernelBuildError("nvcc was not found (looked at $SLEUTH_B200_NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels of sleuth_b200 cannot be built, and there is no other path")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:24]


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("SLEUTH_B200_BUILD_DIR")
    if override:
        return Path(override)
    in_tree = CSRC.parent / "_build"
    if _writable(in_tree):
        return in_tree
    return Path(tempfile.gettempdir()) / f"sleuth_b200_build_{os.getuid()}"


def build(verbose: bool = True) -> Path:
    """Compile the library if it is missing or stale; return its path."""
    out_dir = build_dir()
    out_dir.mkdir(parents=True, exist_ok=True)
    lib = out_dir / LIB_NAME
    stamp = out_dir / "stamp.txt"
    fp = _fingerprint()
    if lib.exists() and stamp.exists() and stamp.read_text().strip() == fp:
        return lib
    nvcc = find_nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call only)")
    t0 = time.time()
    objs = [out_dir / (s.stem + ".o") for s in srcs]

    def compile_one(pair):
        src, obj = pair
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"  compiled {src.name} ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        list(pool.map(compile_one, zip(srcs, objs)))
    tmp = out_dir / (LIB_NAME + f".{os.getpid()}.tmp")
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), "-lcuda"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    stamp.write_text(fp + "\n")
    if verbose:
        _say(f"built {lib.name} in {time.time() - t0:.0f} s")
    return lib


I, L, F, P = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "slb_embed": [P, P, P, I, P, I, I, I, F, P],
    "slb_rmsnorm": [P, P, P, I, P, I, I, F, P],
    "slb_add": [P, P, I, L, P],
    "slb_swiglu": [P, P, I, I, I, P],
    "slb_qkv_post": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "slb_attention_generic": [P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, P],
    "slb_attention_prefill": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P],
    "slb_attention_tc": [P, P, P, P, P, P, P, P, I, I, I, L, L, I, I, I, I, F, P, I, I, P],
    "slb_attention_decode": [P, P, P, P, P, P, P, I, I, I, I, I, I, F, I, P, L, P, L, P, I, P, P, P, P, P, F, P, L, P],
    "slb_gemm_skinny": [P, P, P, I, I, I, I, I, P, L, P, I, P],
    "slb_gemm_skinny_norm": [P, P, F, P, P, I, I, I, I, I, P, L, P, I, P],
    "slb_gemm_tc": [P, P, P, I, I, I, I, I, P, P],
    "slb_tc_wait_probe": [P, I, I, P],
    "slb_decode_layers": [P, P],
    "slb_gemm_tc_qkv": [P, P, I, I, I, I, I, P, P, P, P, P, F, P, P, P, P, P, P, I, P, P],
    "slb_gemm_f32": [P, P, P, P, I, I, I, I, I, I, I, P],
    "slb_penalize": [P, L, I, I, P, P, I, F, P, P, I, P],
    "slb_argmax": [P, L, I, I, P, P, L, P],
    "slb_sample": [P, L, I, I, F, I, F, F, P, P, P],
}


class KernelLibrary:
    """The loaded library. ``call(name, *args)`` runs a launcher and raises on a non-zero return."""

    def __init__(self, path: Path):
        self.path = path
        self.dll = ctypes.CDLL(str(path))
        self.dll.slb_last_error.restype = ctypes.c_char_p
        self._fns = {}
        self.timing = None
        self.launches = 0      # launcher calls made through ``call`` (each starts at least one kernel)
        for name, argtypes in _SIGNATURES.items():
            self.declare(name, argtypes)

    def declare(self, name: str, argtypes) -> None:
        fn = getattr(self.dll, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
        self._fns[name] = fn

    def call(self, name: str, *args) -> None:
        if self.timing is not None:
            return self._timed_call(name, *args)
        rc = self._fns[name](*args)
        self.launches += 1
        if rc != 0:
            raise RuntimeError(self.dll.slb_last_error().decode("utf-8", "replace"))

    # ---- per-launcher device times, for finding where a step's time goes (off unless start_timing was called) ----
    def start_timing(self) -> None:
        self.timing = []

    def stop_timing(self) -> dict:
        """{launcher name: (calls, total milliseconds on the device)}; ends the timing mode."""
        import torch
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.timing or []:
            n, t = out.get(name, (0, 0.0))
            out[name] = (n + 1, t + a.elapsed_time(b))
        self.timing = None
        return out

    def _timed_call(self, name: str, *args) -> None:
        import torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = self._fns[name](*args)
        b.record()
        self.launches += 1
        self.timing.append((name, a, b))
        if rc != 0:
            raise RuntimeError(self.dll.slb_last_error().decode("utf-8", "replace"))


def load() -> KernelLibrary:
    """The kernel library, built on first use. Raises if it cannot be built or loaded."""
    global _lib
    with _lock:
        if _lib is None:
            _lib = KernelLibrary(build())
        return _lib
