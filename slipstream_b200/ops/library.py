"""Compiles the CUDA sources for sm_100a with nvcc and loads them through ctypes.

Libraries are built in the tree (``slipstream_b200/_build``) when that folder can
be written, else in a per-user folder under the system's temporary directory, so
that a fresh checkout works for an ordinary user with an empty HOME.  A library's
file name carries a hash of its sources and flags; a stale one is never loaded.
The attention library is compiled once per head size a model uses, so a first
call compiles only what that model needs.  While nvcc runs, a line is printed to
stderr every few seconds.

There is no fallback: if nvcc is missing or a compile fails, ``KernelBuildError``
says so.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    """The CUDA extension could not be compiled or loaded."""


def _find_nvcc() -> str:
    candidates = [shutil.which("nvcc")]
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    for cand in candidates:
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError(
        "nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda/bin): the CUDA kernels of "
        "slipstream_b200 cannot be compiled and there is no other code path")


def _build_dir() -> Path:
    override = os.environ.get("SLIPSTREAM_B200_BUILD_DIR")
    choices = [Path(override)] if override else []
    choices.append(CSRC.parent / "_build")
    choices.append(Path(tempfile.gettempdir()) / f"slipstream_b200_build_{os.getuid()}")
    for folder in choices:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            fd, probe = tempfile.mkstemp(dir=str(folder), prefix=".probe")
            os.close(fd)
            os.unlink(probe)
            return folder
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {[str(c) for c in choices]}")


def _digest(sources: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for path in sorted(set(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + sources)):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def library_path(name: str, sources: list[str], defines: dict[str, object] | None = None) -> tuple[Path, list[str]]:
    srcs = [CSRC / s for s in sources]
    flags = BASE_FLAGS + ARCH_FLAGS + [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tag = _digest(srcs, flags)
    suffix = "".join(f"_{k.lower()}{v}" for k, v in sorted((defines or {}).items()))
    # look in every candidate folder for an up-to-date build before compiling
    fname = f"lib{name}{suffix}_{tag}.so"
    for folder in (CSRC.parent / "_build", Path(tempfile.gettempdir()) / f"slipstream_b200_build_{os.getuid()}"):
        if (folder / fname).is_file():
            return folder / fname, flags
    return _build_dir() / fname, flags


def compile_library(name: str, sources: list[str], defines: dict[str, object] | None = None,
                    verbose: bool = False) -> Path:
    """Compile (if no up-to-date build exists) and return the .so path."""
    out, flags = library_path(name, sources, defines)
    if out.is_file():
        return out
    nvcc = _find_nvcc()
    tmp = out.with_suffix(f".tmp{os.getpid()}_{threading.get_ident()}.so")
    cmd = [nvcc, *flags, "-I", str(CSRC), "-o", str(tmp), *[str(CSRC / s) for s in sources]]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    label = out.name
    print(f"[slipstream_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            cwd=str(out.parent))
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(5.0):
            print(f"[slipstream_b200] ... still compiling {label} ({time.time() - start:.0f} s)",
                  file=sys.stderr, flush=True)

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    try:
        log, _ = proc.communicate()
    finally:
        done.set()
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed for {label} (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    # builds of earlier sources of the same library are of no further use
    stem = out.name[: -len(out.name.rsplit("_", 1)[1])]
    for old in out.parent.glob(stem + "*.so"):
        if old != out and len(old.name) == len(out.name) and ".tmp" not in old.name:
            old.unlink(missing_ok=True)
    print(f"[slipstream_b200] compiled {label} in {time.time() - start:.1f} s", file=sys.stderr,
          flush=True)
    if verbose and log:
        print(log, file=sys.stderr)
    return out


def load_library(name: str, sources: list[str], defines: dict[str, object] | None = None) -> ctypes.CDLL:
    key = name + repr(sorted((defines or {}).items()))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(name, sources, defines)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelBuildError(f"cannot load {path}: {exc}") from exc
            _loaded[key] = lib
        return lib


def require_cuda() -> None:
    """Fail loudly when there is no GPU to run the kernels on."""
    import torch

    if not torch.cuda.is_available():
        raise KernelBuildError(
            "slipstream_b200 runs on a CUDA device (sm_100a) only; torch.cuda.is_available() is "
            "False and there is no CPU path")
