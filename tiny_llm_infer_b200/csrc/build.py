"""Compiles the CUDA sources of this folder for sm_100a into one shared library.

The library is built in the source tree (``libtllm_kernels.so`` beside the sources),
at the first call that needs it and again whenever a source or a flag changes; a
fingerprint file beside it records what it was built from.  If the tree cannot be
written, ``TLLM_BUILD_DIR`` or a per-user folder under the system's temporary
directory is used instead.  While nvcc runs, a line is printed every few seconds.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path
from typing import List

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libtllm_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=default"]


class BuildError(RuntimeError):
    pass


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def find_nvcc() -> str:
    for cand in (os.environ.get("TLLM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc not found: set TLLM_NVCC or put nvcc on PATH; the CUDA kernels of "
                     "this package have no other implementation")


def fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("TLLM_BUILD_DIR")
    if env:
        return Path(env)
    if _writable(CSRC):
        return CSRC
    return Path(tempfile.gettempdir()) / f"tllm_build_{os.getuid()}"


def library_path(create: bool = True, verbose: bool = True) -> Path:
    """Path of an up-to-date library, building it if needed."""
    out_dir = build_dir()
    lib = out_dir / LIB_NAME
    stamp = out_dir / (LIB_NAME + ".fingerprint")
    want = fingerprint()
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == want:
        return lib
    if not create:
        raise BuildError(f"{lib} is missing or out of date")
    _build(out_dir, lib, stamp, want, verbose)
    return lib


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[tllm build] {msg}", file=sys.stderr, flush=True)


def _build(out_dir: Path, lib: Path, stamp: Path, want: str, verbose: bool) -> None:
    nvcc = find_nvcc()
    if not _writable(out_dir):
        raise BuildError(f"cannot write the kernel library to {out_dir}; set TLLM_BUILD_DIR")
    obj_dir = out_dir / "_build"
    obj_dir.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {lib}", verbose)
    start = time.time()
    jobs = []
    for src in srcs:
        obj = obj_dir / (src.stem + f".{os.getpid()}.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        jobs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    last = time.time()
    pending = list(jobs)
    failed = []
    while pending:
        still = []
        for src, obj, proc in pending:
            if proc.poll() is None:
                still.append((src, obj, proc))
                continue
            out = proc.stdout.read().decode(errors="replace")
            if proc.returncode != 0:
                failed.append((src, out))
            else:
                _say(f"compiled {src.name} ({time.time() - start:.0f} s)", verbose)
        pending = still
        if pending:
            time.sleep(0.2)
            if time.time() - last > 5:
                names = ", ".join(s.name for s, _, _ in pending)
                _say(f"still compiling {names} ({time.time() - start:.0f} s)", verbose)
                last = time.time()
    if failed:
        text = "\n".join(f"--- {s.name} ---\n{o}" for s, o in failed)
        raise BuildError(f"nvcc failed:\n{text}")
    tmp_lib = out_dir / f".{LIB_NAME}.{os.getpid()}"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *[str(o) for _, o, _ in jobs],
           "-lcudart"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    if res.returncode != 0:
        raise BuildError("linking failed:\n" + res.stdout.decode(errors="replace"))
    os.replace(tmp_lib, lib)           # atomic: a concurrent builder cannot leave half a file
    stamp.write_text(want + "\n")
    for _, obj, _ in jobs:
        try:
            obj.unlink()
        except OSError:
            pass
    _say(f"done in {time.time() - start:.0f} s", verbose)


if __name__ == "__main__":
    print(library_path())
