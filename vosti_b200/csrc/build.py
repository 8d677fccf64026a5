"""Compile the CUDA sources of this folder for sm_100a into one shared library.

The library is built in-tree (``csrc/_build/``) the first time it is needed and
whenever a source changed; a folder that cannot be written falls back to a
per-user temporary folder. Progress is printed while nvcc runs because a first
call may take a minute.
"""
from __future__ import annotations

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

HERE = Path(__file__).resolve().parent
LIB_NAME = "libvosti_b200_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _say(message: str) -> None:
    print(f"[vosti_b200] {message}", file=sys.stderr, flush=True)


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for path in sorted(list(HERE.glob("*.cu")) + list(HERE.glob("*.cuh")) + list(HERE.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise RuntimeError("vosti_b200 needs nvcc to compile its sm_100a kernels and found none "
                       "(looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc)")


def _build_dir() -> Path:
    preferred = HERE / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"vosti_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def library_path(build: bool = True, verbose: bool = True) -> Path:
    """Path of an up-to-date library; compiles what is missing when `build`."""
    out_dir = _build_dir()
    lib, stamp = out_dir / LIB_NAME, out_dir / "stamp.txt"
    digest = _digest()
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return lib
    if not build:
        raise RuntimeError(f"{lib} is missing or stale and building was not allowed")
    nvcc = find_nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} (first call only)")
    started = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - started:.0f} s")

    if verbose:
        threading.Thread(target=heartbeat, daemon=True).start()

    def compile_one(src: Path) -> Path:
        obj = out_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{result.stdout}\n{result.stderr}")
        if verbose:
            _say(f"compiled {src.name} ({time.time() - started:.0f} s)")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objects = list(pool.map(compile_one, srcs))
        tmp = out_dir / (LIB_NAME + f".tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objects], "-gencode",
               "arch=compute_100a,code=sm_100a"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"linking {LIB_NAME} failed:\n{result.stdout}\n{result.stderr}")
        os.replace(tmp, lib)
        stamp.write_text(digest)
    finally:
        done.set()
    if verbose:
        _say(f"built {lib.name} in {time.time() - started:.0f} s")
    return lib


HOST_LIB_NAME = "libvosti_b200_host.so"


def host_library_path(verbose: bool = True) -> Path:
    """The C++ host core (no CUDA in it), compiled with g++ on first use."""
    out_dir = _build_dir()
    lib, stamp = out_dir / HOST_LIB_NAME, out_dir / "host_stamp.txt"
    sources = sorted((HERE / "host").glob("*.cpp"))
    h = hashlib.sha256()
    for path in sources:
        h.update(path.read_bytes())
    digest = h.hexdigest()
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return lib
    compiler = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not compiler:
        raise RuntimeError("vosti_b200 needs a C++ compiler (g++) for its host core and found none")
    if verbose:
        _say(f"compiling the C++ host core into {out_dir}")
    tmp = out_dir / (HOST_LIB_NAME + f".tmp{os.getpid()}")
    cmd = [compiler, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-o", str(tmp),
           *[str(s) for s in sources]]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"compiling the host core failed:\n{result.stdout}\n{result.stderr}")
    os.replace(tmp, lib)
    stamp.write_text(digest)
    return lib


if __name__ == "__main__":
    print(library_path())
    print(host_library_path())
