"""Compile the sm_100a kernels with nvcc into shared libraries, at first use.

The sources under ``tokenmill_b200/csrc`` have no dependency beyond the CUDA toolkit (no torch or
pybind headers), so a cold build takes well under a minute. They form five libraries, each built when a
kernel of it is first called, so that a model compiles what it runs and no more: ``main`` (everything the
Qwen2 path, the sampler and the shape-generic kernels need), ``hybrid`` (the kernels of latent attention,
state-space layers, routed experts, 32-bit pair norms), ``gated`` (gated convolutional blocks, windowed attention
with a sink, matrix memory), ``streams`` (several residual streams behind a norm, the selective scan, linear
attention with a decay, and the files of the other two whose kernels such a model also runs) and ``delta`` (matrix
memories with a decay per token and the delta rule, short convolutions with carried inputs, and the files of the others
that a model of such layers beside windowed attention and routed experts runs). A file may be part
of several libraries; the 32-bit matrix product is in all.
A library is written next to the
sources (``csrc/_build``) when that folder can be written, else under the system's temporary folder;
its name carries a hash of the sources and flags, so an edited source is rebuilt and a stale library
is never loaded. While nvcc runs, a line is printed to stderr every few seconds.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# Precise math (no --use_fast_math): division, sqrt and expf keep their IEEE / documented accuracy.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); the "
                           "engine has no path that runs without its compiled sm_100a kernels")


# Files of the ``hybrid`` and ``gated`` libraries; ``main`` is every other .cu file. SHARED files are compiled into all.
HYBRID = ("norm_pair.cu", "latent_attention.cu", "latent_attention_mma_bf16.cu", "ssm_scan.cu", "routed_ffn.cu")
GATED = ("gated_block.cu", "sink_attention.cu", "sink_attention_mma_bf16.cu", "matrix_memory.cu")
STREAMS = ("stream_norm.cu", "selective_scan.cu", "decay_memory.cu", "routed_ffn.cu", "ssm_scan.cu", "sink_attention.cu",
           "sink_attention_mma_bf16.cu", "gated_block.cu")
DELTA = ("gated_memory.cu", "stream_norm.cu", "sink_attention.cu", "sink_attention_mma_bf16.cu", "gated_block.cu",
         "routed_ffn.cu")
SHARED = ("gemm_f32.cu",)
GROUPS = ("main", "hybrid", "gated", "streams", "delta")
_PREFIX = {"main": "libtokenmill_kernels_", "hybrid": "libtokenmill_hybrid_", "gated": "libtokenmill_gated_",
           "streams": "libtokenmill_streams_", "delta": "libtokenmill_delta_"}
_FILES = {"hybrid": HYBRID, "gated": GATED, "streams": STREAMS, "delta": DELTA}


def sources(group: str = "main") -> list[Path]:
    if group not in GROUPS:
        raise KernelBuildError(f"unknown kernel library {group!r}; known: {GROUPS}")
    files = sorted(CSRC.glob("*.cu"))
    if group in _FILES:
        return [f for f in files if f.name in _FILES[group] or f.name in SHARED]
    return [f for f in files if not any(f.name in names for names in _FILES.values())]


def _digest(files: list[Path]) -> str:
    h = hashlib.sha256()
    for f in files + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> Path:
    override = os.environ.get("TOKENMILL_BUILD_DIR")
    cands = [Path(override)] if override else []
    cands += [CSRC / "_build", Path(tempfile.gettempdir()) / f"tokenmill_b200_build_{os.getuid()}"]
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".write_probe_{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for the kernel library (tried {[str(c) for c in cands]})")


def library_path(group: str = "main") -> Path:
    """Where the library for the present sources lives (it may not be built yet)."""
    return _build_dir() / f"{_PREFIX[group]}{_digest(sources(group))}.so"


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}")


def build_all(verbose: bool = True, force: bool = False) -> list[Path]:
    """Build every library (the build check; a run builds only what it calls)."""
    return [build(verbose, force, group) for group in GROUPS]


def build(verbose: bool = True, force: bool = False, group: str = "main") -> Path:
    """Build the library if it is missing; return its path."""
    files = sources(group)
    if not files:
        raise KernelBuildError(f"no .cu sources in {CSRC}")
    out_dir = _build_dir()
    lib = out_dir / f"{_PREFIX[group]}{_digest(files)}.so"
    if lib.exists() and not force:
        return lib
    nvcc = find_nvcc()
    obj_dir = out_dir / f"obj_{lib.stem}_{os.getpid()}"
    obj_dir.mkdir(parents=True, exist_ok=True)
    t0 = time.time()
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(5.0):
            print(f"[tokenmill_b200] compiling sm_100a kernels ({group}: {len(files)} files) ... {time.time() - t0:.0f} s",
                  file=sys.stderr, flush=True)

    if verbose:
        print(f"[tokenmill_b200] compiling sm_100a kernels ({group}: {len(files)} files) into {lib}", file=sys.stderr,
              flush=True)
        threading.Thread(target=heartbeat, daemon=True).start()
    try:
        objs = [obj_dir / (f.stem + ".o") for f in files]
        with ThreadPoolExecutor(max_workers=min(8, len(files))) as pool:
            jobs = [pool.submit(_run, [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(f), "-o", str(o)])
                    for f, o in zip(files, objs)]
            for j in jobs:
                j.result()
        tmp = out_dir / f".{lib.name}.{os.getpid()}.tmp"
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in objs], "-lcuda", "-ldl"])
        os.replace(tmp, lib)  # atomic: a concurrent builder never sees half a library
        for stale in out_dir.glob(_PREFIX[group] + "*.so"):         # libraries of earlier source states
            if stale != lib:
                stale.unlink(missing_ok=True)   # a process that has one mapped keeps its copy
    finally:
        done.set()
        shutil.rmtree(obj_dir, ignore_errors=True)
    if verbose:
        print(f"[tokenmill_b200] kernels built in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return lib
