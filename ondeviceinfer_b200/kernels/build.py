"""Compiling the CUDA sources under ``csrc/`` for sm_100a and loading them.

Each ``.cu`` file becomes one shared library, built with ``nvcc`` the first time it is
needed and reused afterwards.  The file name of a built library carries a hash of the
source, the shared header, the defines and the compiler flags, so an edited source is
never served by a stale build.  Libraries live in ``ondeviceinfer_b200/csrc/_build``
when that folder can be written, else in a per-user folder of the temporary directory;
no home directory and no network are needed.

A model compiles only what it needs (for instance the attention kernels for its own
head size); :func:`build_all` compiles every source, for the packaging check.
While ``nvcc`` runs, a line is printed to stderr every few seconds.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shlex
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Dict, Mapping, Optional

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]

_loaded: Dict[tuple, ctypes.CDLL] = {}
_lock = threading.Lock()

# Extra nvcc flags per source (libraries to link and the like).
EXTRA_FLAGS: Dict[str, list] = {}


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for candidate in (os.environ.get("ODI_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise KernelBuildError("nvcc was not found (PATH, /usr/local/cuda/bin, or $ODI_NVCC); the CUDA kernels "
                           "of ondeviceinfer_b200 cannot be built and there is no fallback path")


def build_dir() -> Path:
    override = os.environ.get("ODI_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    uid = os.getuid() if hasattr(os, "getuid") else 0
    candidates.append(Path(tempfile.gettempdir()) / f"ondeviceinfer_b200-build-{uid}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".probe-{os.getpid()}-{threading.get_ident()}"      # threads may probe side by side
            probe.write_text("")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {[str(c) for c in candidates]}")


def _key(source: Path, defines: Mapping[str, object], extra: list) -> str:
    h = hashlib.sha256()
    h.update(source.read_bytes())
    for header in sorted(CSRC.glob("*.cuh")):
        h.update(header.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(ARCH_FLAGS + BASE_FLAGS + extra).encode())
    return h.hexdigest()[:16]


def _extra_flags(name: str, extra: Optional[list]) -> list:
    """The source's own extra flags plus what ``ODI_NVCC_FLAGS_<NAME>`` adds (for sweeps of build-time constants)."""
    return list(extra or []) + shlex.split(os.environ.get(f"ODI_NVCC_FLAGS_{name.upper()}", ""))


def library_path(name: str, defines: Optional[Mapping[str, object]] = None, extra: Optional[list] = None) -> Path:
    defines, extra = dict(defines or {}), _extra_flags(name, extra)
    source = CSRC / f"{name}.cu"
    if not source.exists():
        raise KernelBuildError(f"no kernel source {source}")
    tag = "".join(f"_{k}{v}" for k, v in sorted(defines.items()))
    return build_dir() / f"libodi_{name}{tag}_{_key(source, defines, extra)}.so"


def compile_library(name: str, defines: Optional[Mapping[str, object]] = None, extra: Optional[list] = None,
                    verbose: bool = True) -> Path:
    """Build ``csrc/<name>.cu`` unless an up-to-date build exists; return the library's path."""
    defines = dict(defines or {})
    out = library_path(name, defines, extra)
    extra = _extra_flags(name, extra)
    if out.exists():
        return out
    source = CSRC / f"{name}.cu"
    tmp = out.with_suffix(f".tmp{os.getpid()}_{threading.get_ident()}.so")      # two builders of one library never share it
    cmd = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *extra, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
           "-I", str(CSRC), str(source), "-o", str(tmp)]
    label = name + "".join(f" {k}={v}" for k, v in sorted(defines.items()))
    if verbose:
        print(f"[ondeviceinfer_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def _progress():
        while not done.wait(10.0):
            if verbose:
                print(f"[ondeviceinfer_b200] still compiling {label} ({time.time() - start:.0f} s)",
                      file=sys.stderr, flush=True)

    ticker = threading.Thread(target=_progress, daemon=True)
    ticker.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        if tmp.exists():
            tmp.unlink()
        raise KernelBuildError(f"nvcc failed for {source.name} ({' '.join(cmd)}):\n{log}")
    os.replace(tmp, out)  # atomic: concurrent builders produce identical files
    if verbose:
        print(f"[ondeviceinfer_b200] built {out.name} in {time.time() - start:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(name: str, defines: Optional[Mapping[str, object]] = None) -> ctypes.CDLL:
    """The loaded library of ``csrc/<name>.cu`` (built on first use, then memoised)."""
    memo = (name, tuple(sorted((defines or {}).items())))
    lib = _loaded.get(memo)
    if lib is not None:
        return lib
    with _lock:
        if memo not in _loaded:
            path = compile_library(name, defines, EXTRA_FLAGS.get(name))
            try:
                _loaded[memo] = ctypes.CDLL(str(path))
            except OSError as error:
                raise KernelBuildError(f"cannot load {path}: {error}") from error
        return _loaded[memo]


# Every source with the defines its default build uses.
# Every library that build_all() makes: the sources without a head size, and the attention kernels for the head
# sizes that the Qwen3 sizes use (128) and that the tests use; any other head size in steps of 16 is compiled
# when a model first needs it.
_HEAD_SIZES_MMA = (16, 32, 48, 64, 80, 96, 112, 128, 192, 256)
ALL_SOURCES = {
    "elementwise": [{}],
    "gemm_f32": [{}],
    "sampling": [{}],
    "gemm_tcgen05": [{}, {"ODI_WAIT_CYCLES": 20_000_000}],      # the second: ops.selftest_bounded_wait
    "gemm_prefill_tcgen05": [{}],
    "attention_simt": [{"ODI_HEAD_DIM": d} for d in _HEAD_SIZES_MMA + (512,)],
    "attention_mma": [{"ODI_HEAD_DIM": d} for d in _HEAD_SIZES_MMA],
    "attention_tcgen05": [{"ODI_HEAD_DIM": 64}, {"ODI_HEAD_DIM": 128}],
}


def build_all(verbose: bool = True, jobs: Optional[int] = None) -> list:
    """Compile every library of ALL_SOURCES that has no up-to-date build, several at a time."""
    from concurrent.futures import ThreadPoolExecutor

    work = [(name, defines) for name, variants in ALL_SOURCES.items() for defines in variants]
    with ThreadPoolExecutor(jobs or min(8, os.cpu_count() or 1)) as pool:
        return list(pool.map(lambda w: compile_library(w[0], w[1], EXTRA_FLAGS.get(w[0]), verbose=verbose), work))
