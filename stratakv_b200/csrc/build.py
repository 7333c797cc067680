"""Compiles the sm_100a kernel library with nvcc and returns the path of the .so.

One library serves one compute dtype and one head size (the attention kernels
keep a head in registers, so the head size is a compile-time constant).  An
engine therefore compiles only what its model needs, at first use, in a build
folder inside the package (or, if that is not writable, under the system's
temporary folder).  The file name carries a hash of the sources and flags, so
a stale library is never loaded.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent
SOURCES = ("elementwise.cu", "linear.cu", "gemm_tcgen05.cu", "attention.cu", "attention_decode.cu", "attention_decode_fused.cu", "attention_prefill.cu", "attention_prefill_tc.cu", "sampling.cu")
HEADERS = ("common.cuh",)
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
COMMON_FLAGS = ("-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden")
DTYPE_CODES = {"float32": 0, "bfloat16": 1}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        candidates.append(Path(found))
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for candidate in candidates:
        if candidate.is_file():
            return str(candidate)
    raise BuildError("nvcc not found (looked in CUDA_HOME, PATH and /usr/local/cuda): "
                     "the kernel library cannot be compiled and there is no other backend")


def _source_hash(flags) -> str:
    digest = hashlib.sha256()
    for name in HEADERS + SOURCES:
        digest.update(name.encode())
        digest.update((CSRC / name).read_bytes())
    digest.update(" ".join(flags).encode())
    return digest.hexdigest()[:12]


def _build_dir() -> Path:
    preferred = CSRC / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"stratakv_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def library_name(dtype: str, head_dim: int) -> str:
    defines = (f"-DSKV_DTYPE={DTYPE_CODES[dtype]}", f"-DSKV_HEAD_DIM={head_dim}")
    flags = ARCH_FLAGS + COMMON_FLAGS + defines
    short = "f32" if dtype == "float32" else "bf16"
    return f"libstratakv_{short}_hd{head_dim}_{_source_hash(flags)}.so"


def find_built(dtype: str, head_dim: int):
    name = library_name(dtype, head_dim)
    for folder in (CSRC / "_build", Path(tempfile.gettempdir()) / f"stratakv_b200_build_{os.getuid()}"):
        if (folder / name).is_file():
            return folder / name
    return None


def build_library(dtype: str, head_dim: int, verbose: bool = True) -> Path:
    """Path of the library for (dtype, head size); compiled now if it is not there yet."""
    if dtype not in DTYPE_CODES:
        raise BuildError(f"no kernels for dtype {dtype}")
    if head_dim <= 0 or head_dim % 16 != 0 or head_dim > 256:
        raise BuildError(f"head size {head_dim} is not supported: the kernels take multiples of 16 up to 256")
    built = find_built(dtype, head_dim)
    if built is not None:
        return built
    nvcc = find_nvcc()
    folder = _build_dir()
    target = folder / library_name(dtype, head_dim)
    lock_path = folder / (target.name + ".lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if target.is_file():
                return target
            _compile(nvcc, dtype, head_dim, target, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return target


def _compile(nvcc: str, dtype: str, head_dim: int, target: Path, verbose: bool) -> None:
    defines = (f"-DSKV_DTYPE={DTYPE_CODES[dtype]}", f"-DSKV_HEAD_DIM={head_dim}")
    start = time.time()
    say = (lambda text: print(f"[stratakv_b200] {text}", file=sys.stderr, flush=True)) if verbose else (lambda text: None)
    say(f"compiling kernels for sm_100a ({dtype}, head size {head_dim}); this happens once")
    done = threading.Event()

    def heartbeat():
        while not done.wait(5.0):
            say(f"still compiling ({time.time() - start:.0f} s)")

    ticker = threading.Thread(target=heartbeat, daemon=True)
    ticker.start()
    work = Path(tempfile.mkdtemp(prefix="skv_build_", dir=str(target.parent)))
    try:
        jobs = []
        for name in SOURCES:
            obj = work / (name + ".o")
            cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *defines, "-I", str(CSRC), "-c", str(CSRC / name), "-o", str(obj)]
            jobs.append((name, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects = []
        for name, obj, proc in jobs:
            output, _ = proc.communicate()
            if proc.returncode != 0:
                raise BuildError(f"nvcc failed on {name}:\n{output}")
            objects.append(str(obj))
        staged = work / target.name
        link = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(staged), *objects],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if link.returncode != 0:
            raise BuildError(f"nvcc failed to link {target.name}:\n{link.stdout}")
        os.replace(staged, target)
    finally:
        done.set()
        shutil.rmtree(work, ignore_errors=True)
    say(f"kernels ready in {time.time() - start:.0f} s: {target.name}")
