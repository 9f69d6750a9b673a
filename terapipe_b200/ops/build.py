"""In-tree build of the native libraries.

* ``_tp_sm100.so``  — CUDA kernels, compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); cross-compiles on machines without a GPU.
* ``_tp_sm100_checked.so`` — the same sources compiled with ``-DTP_CHECKED``: index checks next
  to every raw-pointer access into peer staging, flag and statistics arrays; a failed check
  writes a code into the launch's status word and skips the access.  Loaded instead of the
  regular library when ``TERAPIPE_CHECKED=1``.
* ``_tp_host.so``   — host C++ (slice-schedule dynamic program), compiled by g++.

The libraries sit beside this file so that a source checkout carries them to wherever the
checkout is copied; nothing is installed into site-packages and there is no JIT cache.
A stamp file holds a hash of the sources so unchanged sources are not rebuilt.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
CUDA_LIB = HERE / "_tp_sm100.so"
CUDA_LIB_CHECKED = HERE / "_tp_sm100_checked.so"
HOST_LIB = HERE / "_tp_host.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-shared"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _stale(lib: Path, sources) -> bool:
    stamp = lib.with_suffix(".stamp")
    return not (lib.exists() and stamp.exists() and stamp.read_text() == _digest(sources))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}")
    return res.stdout + res.stderr


def cuda_sources():
    return sorted(CSRC.glob("*.cu"))


def build_cuda(force=False, verbose=False, ptxas_info=False, checked=False) -> Path:
    lib = CUDA_LIB_CHECKED if checked else CUDA_LIB
    srcs = cuda_sources()
    deps = srcs + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    if not force and not _stale(lib, deps):
        return lib
    objs = []
    build_dir = HERE / ("build_checked" if checked else "build")
    build_dir.mkdir(exist_ok=True)
    procs = []
    flags = [f for f in NVCC_FLAGS if f != "-shared"]
    if checked:
        flags += ["-DTP_CHECKED"]
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    for src in srcs:
        obj = build_dir / (src.stem + ".o")
        cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(map(str, cmd)), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                            text=True)))
        objs.append(obj)
    log = ""
    for cmd, proc in procs:
        out, _ = proc.communicate()
        log += out
        if proc.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}")
    # link beside the target and rename: a reader (or a copy of the tree) never sees half a library
    tmp = lib.with_suffix(".so.tmp")
    _run([_nvcc(), "-shared", "-Xcompiler", "-fPIC", "-o", str(tmp), *map(str, objs)], verbose)
    os.replace(tmp, lib)
    lib.with_suffix(".stamp").write_text(_digest(deps))
    if ptxas_info:
        print(log)
    return lib


def build_host(force=False, verbose=False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    deps = srcs + [CSRC / "tile_order.h"]      # shared with the kernels, walked by the host tests
    if not force and not _stale(HOST_LIB, deps):
        return HOST_LIB
    tmp = HOST_LIB.with_suffix(".so.tmp")
    _run(["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-o", str(tmp), *map(str, srcs)], verbose)
    os.replace(tmp, HOST_LIB)
    HOST_LIB.with_suffix(".stamp").write_text(_digest(deps))
    return HOST_LIB


def build_all(force=False, verbose=False, checked=True):
    """Host library, kernel library and (unless ``checked=False``) the checked kernel library."""
    out = (build_host(force, verbose), build_cuda(force, verbose))
    if checked:
        out += (build_cuda(force, verbose, checked=True),)
    return out


if __name__ == "__main__":
    print("built", *build_all(force="--force" in sys.argv, verbose=True))
