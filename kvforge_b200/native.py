"""Builds the CUDA sources under ``csrc/`` with nvcc for sm_100a and loads them with ctypes.

The kernels are plain ``extern "C"`` launchers that take device pointers and a stream, so
they need no torch headers and a source file compiles in seconds.  A library is built at
its first use, into ``csrc/_build/<hash>/`` inside the package when that is writable and
otherwise into a per-user folder under the system temp directory; the hash covers the
sources, the headers and the flags, so an edited source rebuilds and an unchanged one is
loaded as it is.  While nvcc runs, a progress line goes to stderr every few seconds.

There is no fallback: if nvcc is missing or a source fails to compile, ``load`` raises.
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
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# name -> (sources, extra flags).  One shared library per entry.
LIBRARIES: dict[str, tuple[list[str], list[str]]] = {
    "core": (
        ["elementwise.cu", "gemm_f32.cu", "attention_generic.cu", "attention_mma.cu", "attention_decode_tma.cu", "attention_tcgen05.cu", "gemm_skinny_bf16.cu", "gemm_tcgen05_bf16.cu", "sampling.cu"],
        [],
    ),
    # one entry point that allocates nothing (csrc/kvforge_noalloc.h); a library of its own, so
    # that only a process that asks for it holds its built-in scratch array
    "noalloc": (["attention_decode_noalloc.cu"], []),
}

_loaded: dict[str, ctypes.CDLL] = {}


class NativeBuildError(RuntimeError):
    pass


def register_library(name: str, sources: list[str], flags: list[str] | None = None) -> None:
    """Declare a further library of ``csrc`` sources (built on first ``load(name)``)."""
    LIBRARIES[name] = (list(sources), list(flags or []))


def find_nvcc() -> str:
    for cand in (
        os.environ.get("KVFORGE_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise NativeBuildError("nvcc not found (looked at KVFORGE_NVCC, PATH, CUDA_HOME, /usr/local/cuda)")


def _digest(name: str) -> str:
    sources, flags = LIBRARIES[name]
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + flags).encode())
    # every source and header: a source may include another (the hash errs on the side of rebuilding)
    for f in sorted({p.name for pat in ("*.cu", "*.cuh", "*.h") for p in CSRC.glob(pat)} | set(sources)):
        h.update(f.encode())
        h.update((CSRC / f).read_bytes())
    return h.hexdigest()[:16]


def _build_root() -> Path:
    env = os.environ.get("KVFORGE_BUILD_DIR")
    if env:
        root = Path(env)
        root.mkdir(parents=True, exist_ok=True)
        return root
    root = CSRC / "_build"
    try:
        root.mkdir(parents=True, exist_ok=True)
        probe = root / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return root
    except OSError:
        root = Path(tempfile.gettempdir()) / f"kvforge_b200-build-{os.getuid()}"
        root.mkdir(parents=True, exist_ok=True)
        return root


def library_path(name: str) -> Path:
    return _build_root() / f"{name}-{_digest(name)}" / f"libkvforge_b200_{name}.so"


def _say(msg: str) -> None:
    print(f"[kvforge_b200] {msg}", file=sys.stderr, flush=True)


def build(name: str, verbose: bool = True) -> Path:
    """Compile library ``name`` if its ``.so`` is not there yet; returns the path."""
    out = library_path(name)
    if out.is_file():
        return out
    out.parent.mkdir(parents=True, exist_ok=True)
    lock_path = out.parent / ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if out.is_file():  # another process built it while we waited
                return out
            nvcc = find_nvcc()
            sources, flags = LIBRARIES[name]
            t0 = time.time()
            if verbose:
                _say(f"compiling {len(sources)} CUDA sources of '{name}' for sm_100a (first use) ...")
            procs = []
            for src in sources:
                obj = out.parent / (Path(src).stem + ".o")
                cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *flags, "-I", str(CSRC), "-c", str(CSRC / src), "-o", str(obj)]
                procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
            pending = list(procs)
            last = time.time()
            while pending:
                pending = [p for p in pending if p[2].poll() is None]
                if pending and verbose and time.time() - last > 5:
                    last = time.time()
                    _say(f"  still compiling {', '.join(p[0] for p in pending)} ({time.time() - t0:.0f} s)")
                time.sleep(0.05)
            for src, _, proc in procs:
                log = proc.stdout.read() if proc.stdout else ""
                if proc.returncode != 0:
                    raise NativeBuildError(f"nvcc failed on {src}:\n{log}")
            tmp = out.with_suffix(".so.tmp")
            cmd = [nvcc, "-shared", *ARCH_FLAGS, "-o", str(tmp), *[str(o) for _, o, _ in procs]]
            res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if res.returncode != 0:
                raise NativeBuildError(f"link of '{name}' failed:\n{res.stdout}")
            os.replace(tmp, out)
            if verbose:
                _say(f"built {out.name} in {time.time() - t0:.0f} s")
            _prune_stale(name, out.parent)
            return out
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _prune_stale(name: str, keep: Path) -> None:
    """Builds of ``name`` from sources that have changed since are of no use to anyone."""
    for old in keep.parent.glob(f"{name}-*"):
        if old != keep and old.is_dir():
            shutil.rmtree(old, ignore_errors=True)


def load(name: str = "core") -> ctypes.CDLL:
    """The loaded library ``name`` (built first if needed)."""
    lib = _loaded.get(name)
    if lib is None:
        path = build(name)
        lib = ctypes.CDLL(str(path))
        _loaded[name] = lib
    return lib


def build_all(verbose: bool = True) -> list[Path]:
    return [build(name, verbose) for name in LIBRARIES]
