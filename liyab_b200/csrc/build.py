"""Builds and loads the engine's library and its two programs.

Every .cu file of this folder (the kernels) is compiled for sm_100a with nvcc and
every .cpp file of ../host (the C++20 host: configuration, weights, cache manager,
step function, scheduler, engine, C interface) with the host compiler; the objects
are linked into libliyab_b200.so under `_build/` beside the sources (or, where
that folder cannot be written, under the system's temporary folder), and the
programs liyab-cli and trace_run (../host/tools) are linked against it.  Nothing
is built when what is on disk was made from the same sources and flags.  The first
call in a fresh checkout therefore compiles what the engine needs, printing a line
per file; later calls only load.

There is no fallback: without the library (no nvcc, a compile error) the engine
raises, it never computes on the CPU or through another library instead.
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
from typing import List, Optional

from ..status import backend_error

HERE = os.path.dirname(os.path.abspath(__file__))
HOST = os.path.join(os.path.dirname(HERE), "host")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB_NAME = "libliyab_b200.so"
PROGRAMS = ("liyab_cli", "trace_run")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-warn-spills"]
CXX_FLAGS = ["-std=c++20", "-O2", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter"]
# LIYAB_B200_SANITIZE=address,undefined builds the C++ host with those sanitizers into a folder of its own
# (`_build_sanitize`); the process that loads it needs the sanitizer's runtime first (LD_PRELOAD=libasan.so for Python).
SANITIZE = os.environ.get("LIYAB_B200_SANITIZE", "")
if SANITIZE:
    CXX_FLAGS = CXX_FLAGS + [f"-fsanitize={SANITIZE}", "-fno-omit-frame-pointer", "-g", "-O1"]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def _say(msg: str) -> None:
    print(f"[liyab_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    """The CUDA sources (names in this folder) and the host sources (paths relative to this folder)."""
    cu = sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))
    cpp = sorted(os.path.join("..", "host", f) for f in os.listdir(HOST) if f.endswith(".cpp"))
    return cu + cpp


def _headers() -> List[str]:
    own = sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))
    host = sorted(os.path.join("..", "host", f) for f in os.listdir(HOST) if f.endswith(".h"))
    public = sorted(os.path.join("..", "include", f) for f in os.listdir(INCLUDE) if f.endswith(".h"))
    return own + host + public


def _digest(files: List[str], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for name in files:
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(name.encode() + b"\0" + f.read())
    return h.hexdigest()[:24]


def find_cxx() -> str:
    for cand in (os.environ.get("LIYAB_CXX"), os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++")):
        if cand and shutil.which(cand):
            return shutil.which(cand)
    raise backend_error("no C++ compiler was found (looked at $LIYAB_CXX, $CXX, g++ and c++ on PATH); the engine's host "
                        "library cannot be built")


def cuda_include(nvcc: str) -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "include")


def find_nvcc() -> str:
    for cand in (os.environ.get("LIYAB_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise backend_error("nvcc was not found (looked at $LIYAB_NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin); "
                        "the engine's kernels cannot be built and there is no other path")


def build_dir() -> str:
    env = os.environ.get("LIYAB_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    local = os.path.join(HERE, "_build_sanitize" if SANITIZE else "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".write_probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return local
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"liyab_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _compile_one(nvcc: str, src: str, obj: str, log: str) -> None:
    if src.endswith(".cu"):
        cmd = [nvcc, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    else:
        cmd = [find_cxx(), *CXX_FLAGS, "-I", cuda_include(nvcc), "-c", os.path.join(HERE, src), "-o", obj]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        raise backend_error(f"{os.path.basename(cmd[0])} failed on {src}:\n{proc.stdout[-4000:]}")


def ensure_built(verbose: bool = True) -> str:
    """Compiles what is out of date and returns the path of the library."""
    out = build_dir()
    srcs, hdrs = sources(), _headers()
    flags = " ".join(NVCC_FLAGS + CXX_FLAGS)
    whole = _digest(srcs + hdrs, flags)
    lib = os.path.join(out, LIB_NAME)
    stamp = os.path.join(out, "stamp")

    def fresh() -> bool:
        try:
            with open(stamp) as f:
                return (f.read().strip() == whole and os.path.isfile(lib)
                        and all(os.path.isfile(os.path.join(out, p)) for p in PROGRAMS))
        except OSError:
            return False

    if fresh():
        return lib
    with open(os.path.join(out, ".lock"), "w") as lockf:
        fcntl.flock(lockf, fcntl.LOCK_EX)
        try:
            if fresh():
                return lib
            nvcc = find_nvcc()
            # An object's name carries the digest of its source, the headers and its own compiler's flags, so the
            # kernels' objects are the same with and without sanitizers on the host and are taken over from `_build`.
            hdr_digest = {True: _digest(hdrs, " ".join(NVCC_FLAGS)), False: _digest(hdrs, " ".join(CXX_FLAGS))}
            plain_dir = os.path.join(HERE, "_build")
            todo, objs = [], []
            for src in srcs:
                tag = _digest([src], hdr_digest[src.endswith(".cu")])
                name = f"{os.path.splitext(os.path.basename(src))[0]}.{tag}.o"
                obj = os.path.join(out, name)
                objs.append(obj)
                if not os.path.isfile(obj) and out != plain_dir and os.path.isfile(os.path.join(plain_dir, name)):
                    shutil.copyfile(os.path.join(plain_dir, name), obj + f".tmp{os.getpid()}")
                    os.replace(obj + f".tmp{os.getpid()}", obj)
                if not os.path.isfile(obj):
                    todo.append((src, obj))
            if todo and verbose:
                _say(f"compiling {len(todo)} source file(s) (CUDA for sm_100a, C++ host) into {out} (first call only)")
            t0 = time.time()
            done = [0]

            def work(item):
                src, obj = item
                tmp = obj + f".tmp{os.getpid()}"
                _compile_one(nvcc, src, tmp, os.path.join(out, os.path.basename(src) + ".log"))
                os.replace(tmp, obj)
                done[0] += 1
                if verbose:
                    _say(f"  compiled {os.path.basename(src)} ({done[0]}/{len(todo)}, {time.time() - t0:.0f} s)")

            with ThreadPoolExecutor(max_workers=min(8, max(1, os.cpu_count() or 1))) as pool:
                list(pool.map(work, todo))
            tmp_lib = lib + f".tmp{os.getpid()}"
            link = [nvcc, "-shared", "-o", tmp_lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl", "-lpthread"]
            if SANITIZE:         # the host compiler finds its own sanitizer runtimes; nvcc's link line does not
                cuda_lib = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "lib64")
                link = [find_cxx(), "-shared", "-o", tmp_lib, *objs, f"-fsanitize={SANITIZE}", "-L", cuda_lib, "-lcudart_static",
                        "-ldl", "-lpthread", "-lrt"]
            proc = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if proc.returncode != 0:
                raise backend_error(f"linking {LIB_NAME} failed:\n{proc.stdout[-4000:]}")
            os.replace(tmp_lib, lib)
            for prog in PROGRAMS:       # the programs talk to the library through its C interface only
                tmp_prog = os.path.join(out, f"{prog}.tmp{os.getpid()}")
                cmd = [find_cxx(), "-std=c++17", "-O2", os.path.join(HOST, "tools", prog + ".cpp"), "-o", tmp_prog,
                       "-L", out, "-lliyab_b200", "-Wl,-rpath,$ORIGIN"] + ([f"-fsanitize={SANITIZE}"] if SANITIZE else [])
                proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                if proc.returncode != 0:
                    raise backend_error(f"building {prog} failed:\n{proc.stdout[-4000:]}")
                os.replace(tmp_prog, os.path.join(out, prog))
            with open(stamp, "w") as f:
                f.write(whole)
            keep = set(objs)
            for name in os.listdir(out):       # objects of older sources
                path = os.path.join(out, name)
                if name.endswith(".o") and path not in keep:
                    os.unlink(path)
            if verbose and todo:
                _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
            return lib
        finally:
            fcntl.flock(lockf, fcntl.LOCK_UN)


def program(name: str) -> str:
    """The path of a built program (liyab_cli or trace_run); built first if it has to be."""
    return os.path.join(os.path.dirname(ensure_built()), name)


def load_library() -> ctypes.CDLL:
    """The loaded library; built first if it has to be.  Its symbols are visible to plug-ins loaded later."""
    global _lib
    with _lock:
        if _lib is None:
            path = ensure_built()
            try:
                _lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
            except OSError as e:
                raise backend_error(f"cannot load {path}: {e}") from e
        return _lib
