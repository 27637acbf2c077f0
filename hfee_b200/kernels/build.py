"""Compiles the CUDA sources under ``csrc/`` for sm_100a into one shared library.

The library is built on first use (and by ``__graft_entry__.build()``) with nvcc,
one object per source in parallel, into ``hfee_b200/_build/<hash>/`` where the
hash covers the sources and the flags; if the package folder is not writable a
per-user folder under the system temp directory is used.  Progress lines go to
stderr.  No torch headers are involved: the kernels have a plain C interface.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math=false", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]
LIB_NAME = "libhfee_kernels.so"


class KernelBuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[hfee_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("HFEE_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found (looked at $HFEE_NVCC, PATH and /usr/local/cuda/bin); "
                           "the sm_100a kernels cannot be built")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _flags() -> List[str]:
    return ARCH_FLAGS + [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]


def _digest() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(_flags()).encode())
    return h.hexdigest()[:16]


def _build_root() -> str:
    pkg = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    root = os.path.join(pkg, "_build")
    try:
        os.makedirs(root, exist_ok=True)
        probe = os.path.join(root, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return root
    except OSError:
        root = os.path.join(tempfile.gettempdir(), f"hfee_b200-build-{os.getuid()}")
        os.makedirs(root, exist_ok=True)
        return root


def library_path() -> str:
    return os.path.join(_build_root(), _digest(), LIB_NAME)


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    cmd = [nvcc] + _flags() + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
    t0 = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {src}:\n{' '.join(cmd)}\n{proc.stdout}")
    _say(f"compiled {src} ({time.time() - t0:.0f}s)")


def _prune(root: str, keep: str) -> None:
    """Remove builds of older source versions (folders named by another digest)."""
    for name in os.listdir(root):
        path = os.path.join(root, name)
        if name != keep and os.path.isdir(path) and len(name) == 16:
            shutil.rmtree(path, ignore_errors=True)


def build(force: bool = False) -> str:
    """Build the library if it is not there yet; returns its path."""
    out = library_path()
    if os.path.isfile(out) and not force:
        return out
    out_dir = os.path.dirname(out)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(out) and not force:
                return out
            nvcc = _nvcc()
            srcs = sources()
            _say(f"building {len(srcs)} CUDA sources for sm_100a into {out_dir} (first call only)")
            t0 = time.time()
            objs = [os.path.join(out_dir, s[:-3] + ".o") for s in srcs]
            workers = max(1, min(len(srcs), os.cpu_count() or 1))
            with concurrent.futures.ThreadPoolExecutor(workers) as pool:
                futures = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
                pending = set(futures)
                while pending:
                    done, pending = concurrent.futures.wait(pending, timeout=15)
                    for f in done:
                        f.result()
                    if pending:
                        _say(f"still compiling ({len(pending)} of {len(srcs)} sources left, {time.time() - t0:.0f}s)")
            tmp = out + f".{os.getpid()}.tmp"
            cmd = [nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs + ["-lcudart"]
            proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if proc.returncode != 0:
                raise KernelBuildError(f"link failed:\n{' '.join(cmd)}\n{proc.stdout}")
            os.replace(tmp, out)
            _say(f"built {LIB_NAME} in {time.time() - t0:.0f}s")
            _prune(os.path.dirname(out_dir), keep=os.path.basename(out_dir))
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
