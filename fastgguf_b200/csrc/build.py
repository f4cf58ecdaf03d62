"""Compile the CUDA sources of this folder for sm_100a into shared libraries, on first use.

Each *module* is a small group of ``.cu`` files linked into one ``libfg_<module>.so`` that the
Python side loads with ``ctypes``.  A module is compiled when something first asks for it, so
a run compiles what its model and dtype need and nothing else.  The sources include no
framework headers: a file compiles in seconds with plain ``nvcc``.

The libraries are kept beside the sources (``csrc/_build/``) when that folder can be written,
else in a per-user folder under the system's temporary directory; no home directory is needed.
A library is rebuilt when its sources or flags change (content hash).  While compiling, a line
is printed to stderr at the start and every few seconds.
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

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))

#: module name -> source files.  Headers every module depends on are listed in HEADERS.
MODULES = {
    "core": ["elementwise.cu", "gemm_generic.cu", "attention_generic.cu", "sampling.cu"],
    "tc": ["gemm_tc.cu"],
    "attn": ["attention_decode.cu", "attention_prefill.cu", "attention_prefill_tc.cu"],
    # the C++ host: configuration, weights, cache, step function, generation loop, C interface; it opens the
    # kernel libraries above by name when a model first needs them
    "engine": ["host/api.cpp", "host/cache.cpp", "host/config.cpp", "host/device.cpp", "host/model.cpp", "host/parts.cpp",
               "host/runner.cpp", "host/safetensors.cpp", "host/host_kernels.cu"],
}
LINK_FLAGS = {"engine": ["-ldl"]}
HEADERS = ["common.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    cand = [os.environ.get("FASTGGUF_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.exists(c):
            return c
    raise BuildError("nvcc was not found (PATH, /usr/local/cuda/bin, or $FASTGGUF_NVCC); the CUDA kernels "
                     "of fastgguf_b200 cannot be built and there is no fallback path")


def build_dir() -> str:
    """Where libraries are kept: beside the sources if writable, else a per-user temp folder."""
    override = os.environ.get("FASTGGUF_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    local = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"fastgguf_b200-build-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _module_hash(module: str) -> str:
    h = hashlib.sha1()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sorted(MODULES[module] + HEADERS + _extra_headers(module)):
        with open(os.path.join(CSRC_DIR, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    return h.hexdigest()


def _extra_headers(module: str) -> list:
    top = [f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")) and f not in HEADERS]
    if module != "engine":
        return top
    host = os.path.join(CSRC_DIR, "host")
    return top + ["host/" + f for f in os.listdir(host) if f.endswith(".hpp")]


def _say(msg: str) -> None:
    print(f"[fastgguf_b200] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: str, obj: str, extra: list) -> None:
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", CSRC_DIR, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise BuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{p.stdout}\n{p.stderr}")


def build_module(module: str, verbose_ptxas: bool = False) -> str:
    """Build (if stale) and return the path of ``libfg_<module>.so``."""
    if module not in MODULES:
        raise BuildError(f"unknown kernel module '{module}' (known: {', '.join(MODULES)})")
    out_dir = build_dir()
    lib = os.path.join(out_dir, f"libfg_{module}.so")
    stamp = lib + ".hash"
    want = _module_hash(module)

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return f.read().strip() == want and os.path.exists(lib)
        except OSError:
            return False

    if fresh():
        return lib
    with open(os.path.join(out_dir, f".{module}.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if fresh():           # another process built it meanwhile
            return lib
        nvcc = _nvcc()
        srcs = MODULES[module]
        _say(f"compiling kernel module '{module}' for sm_100a ({len(srcs)} files) into {out_dir}")
        t0 = time.time()
        done = threading.Event()

        def ticker():
            while not done.wait(10.0):
                _say(f"still compiling '{module}' ({time.time() - t0:.0f} s)")

        th = threading.Thread(target=ticker, daemon=True)
        th.start()
        try:
            extra = ["-Xptxas", "-v"] if verbose_ptxas else []
            objs = [os.path.join(out_dir, f"{module}-{os.path.splitext(s)[0].replace('/', '_')}.{os.getpid()}.o") for s in srcs]
            with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 2)) as ex:
                list(ex.map(lambda a: _compile_one(nvcc, a[0], a[1], extra), zip(srcs, objs)))
            tmp = lib + f".{os.getpid()}.tmp"
            p = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, *LINK_FLAGS.get(module, [])], capture_output=True, text=True)
            if p.returncode != 0:
                raise BuildError(f"linking {lib} failed:\n{p.stdout}\n{p.stderr}")
            os.replace(tmp, lib)
            with open(stamp, "w") as f:
                f.write(want)
            for o in objs:
                try:
                    os.unlink(o)
                except OSError:
                    pass
        finally:
            done.set()
        _say(f"built '{module}' in {time.time() - t0:.1f} s")
    return lib


_loaded: dict = {}


def load_module(module: str) -> ctypes.CDLL:
    """The loaded library of a module; built first if needed.  Fails loudly, never falls back."""
    lib = _loaded.get(module)
    if lib is None:
        path = build_module(module)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"could not load {path}: {e}") from None
        _loaded[module] = lib
    return lib


def build_all() -> list:
    return [build_module(m) for m in MODULES]


if __name__ == "__main__":
    for path in build_all():
        print(path)
