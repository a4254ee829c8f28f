"""Compile the engine's CUDA sources into one shared library for sm_100a.

nvcc is called directly (one object per ``.cu``, in parallel, then a link); no
Python headers are involved, so a full build takes well under a minute.  The
library is rebuilt when a source, a header or a flag has changed.  It lives in
``csrc/_build/`` inside the package when that is writable, else in a per-user
folder under the system's temporary directory.  While compiling, a line is
printed to stderr for every finished file and every few seconds of waiting.
"""
from __future__ import annotations

import concurrent.futures as cf
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libbinfer_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


# BINFER_B200_TRACE=1: the kernels of the decode step record timestamps (common.cuh, BF_TRACE);
# that library is a build of its own in a folder of its own.
TRACE = os.environ.get("BINFER_B200_TRACE", "0") == "1"
if TRACE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DBF_TRACE"]


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[binfer_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin)")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def build_dir() -> str:
    override = os.environ.get("BINFER_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    local = os.path.join(HERE, "_build_trace" if TRACE else "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(),
                         f"binfer_b200_build{'_trace' if TRACE else ''}_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def lib_path() -> str:
    return os.path.join(build_dir(), LIB_NAME)


def is_current(bdir: str | None = None) -> bool:
    bdir = bdir or build_dir()
    stamp = os.path.join(bdir, "stamp")
    if not (os.path.exists(stamp) and os.path.exists(os.path.join(bdir, LIB_NAME))):
        return False
    with open(stamp) as f:
        return f.read().strip() == _fingerprint()


def _compile_one(nvcc: str, src: str, obj: str, extra: List[str]) -> str:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra, "-I", HERE, "-c",
           os.path.join(HERE, src), "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode:
        raise BuildError(f"nvcc failed on {src}:\n{r.stdout}")
    return r.stdout


def ensure_built(verbose: bool = True, ptxas_info: bool = False) -> str:
    """Build if needed; return the path of the shared library."""
    bdir = build_dir()
    if is_current(bdir):
        return os.path.join(bdir, LIB_NAME)
    with open(os.path.join(bdir, "lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if is_current(bdir):          # another process built it while we waited
            return os.path.join(bdir, LIB_NAME)
        nvcc = find_nvcc()
        srcs = sources()
        t0 = time.time()
        if verbose:
            _log(f"compiling {len(srcs)} CUDA files for sm_100a with {nvcc} into {bdir}")
        extra = ["-Xptxas", "-v"] if ptxas_info else []
        objs = [os.path.join(bdir, s[:-3] + ".o") for s in srcs]
        with cf.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
            futs = {ex.submit(_compile_one, nvcc, s, o, extra): s for s, o in zip(srcs, objs)}
            pending = set(futs)
            while pending:
                done, pending = cf.wait(pending, timeout=5.0)
                for f in done:
                    out = f.result()
                    if verbose:
                        _log(f"  {futs[f]} done ({time.time() - t0:.0f} s)")
                    if ptxas_info and out:
                        print(out, file=sys.stderr)
                if pending and verbose and not done:
                    _log(f"  still compiling {len(pending)} files ({time.time() - t0:.0f} s)")
        tmp = os.path.join(bdir, LIB_NAME + f".tmp{os.getpid()}")
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs],
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode:
            raise BuildError(f"link failed:\n{r.stdout}")
        os.replace(tmp, os.path.join(bdir, LIB_NAME))
        with open(os.path.join(bdir, "stamp"), "w") as f:
            f.write(_fingerprint())
        if verbose:
            _log(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return os.path.join(bdir, LIB_NAME)


if __name__ == "__main__":
    print(ensure_built(verbose=True, ptxas_info="--ptxas" in sys.argv))
