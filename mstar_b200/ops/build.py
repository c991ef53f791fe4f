"""Compile the CUDA and C++ sources of this package into shared libraries.

Libraries are built the first time something needs them and are then found by
the hash of their sources, flags and compiler.  They live in ``csrc/_build``
inside the package when that folder can be written (so a built tree can be
copied to another machine as it is), else in a per-user folder under the
system's temporary directory.  Nothing is written to the home directory.

CUDA sources are compiled for sm_100a only and without fast-math; there is no
other backend and no CPU fallback: if nvcc or the sources are missing, the
error is raised to the caller.
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
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]

# library name -> (kind, sources relative to csrc, extra link flags)
LIBRARIES = {
    "elementwise": ("cuda", ["elementwise.cu"], []),
    "attention_generic": ("cuda", ["attention_generic.cu"], []),
    "attention_decode": ("cuda", ["attention_decode.cu"], []),
    "attention_prefill": ("cuda", ["attention_prefill.cu"], []),
    "attention_prefill_tc": ("cuda", ["attention_prefill_tc.cu"], []),
    "attention_decode_noalloc": ("cuda", ["attention_decode_noalloc.cu"], []),
    "gemm_f32": ("cuda", ["gemm_f32.cu"], []),
    "gemm_smallm_bulk": ("cuda", ["gemm_smallm_bulk.cu"], []),
    "gemm_tcgen05": ("cuda", ["gemm_tcgen05.cu"], []),
    "gemm_skinny": ("cuda", ["gemm_skinny.cu"], []),
    "sampling": ("cuda", ["sampling.cu"], []),
    "host": ("host", ["host/cache_manager.cpp"], []),
}

_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[mstar_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cand = os.environ.get("MSTAR_NVCC") or shutil.which("nvcc")
    if not cand:
        for p in ("/usr/local/cuda/bin/nvcc",):
            if os.path.exists(p):
                cand = p
                break
    if not cand:
        raise BuildError("nvcc not found: the CUDA kernels of mstar_b200 cannot be compiled "
                         "(set MSTAR_NVCC or put nvcc on PATH)")
    return cand


def _compiler_id(kind: str) -> str:
    exe = find_nvcc() if kind == "cuda" else (shutil.which("g++") or "g++")
    try:
        out = subprocess.run([exe, "--version"], capture_output=True, text=True, check=True).stdout
    except (OSError, subprocess.CalledProcessError) as exc:
        raise BuildError(f"cannot run {exe}: {exc}") from exc
    return exe + "\n" + out


def build_dir() -> Path:
    override = os.environ.get("MSTAR_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"mstar_b200_build_{os.getuid()}")
    for d in candidates:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise BuildError("no writable folder for compiled kernels (tried "
                     + ", ".join(str(c) for c in candidates) + ")")


def _with_includes(sources: list) -> list:
    """The sources and, recursively, every file of this tree they #include "..."."""
    import re

    seen: dict = {}
    todo = [CSRC / s for s in sources]
    while todo:
        f = todo.pop()
        if f in seen:
            continue
        if not f.is_file():
            raise BuildError(f"source file {f} is missing")
        text = f.read_text()
        seen[f] = text
        for inc in re.findall(r'^\s*#\s*include\s+"([^"]+)"', text, flags=re.M):
            for base in (f.parent, CSRC):
                if (base / inc).is_file():
                    todo.append((base / inc).resolve())
                    break
    return sorted(seen.items())


def library_hash(name: str) -> str:
    kind, sources, extra = LIBRARIES[name]
    h = hashlib.sha256()
    h.update(_compiler_id(kind).encode())
    h.update(" ".join((NVCC_FLAGS if kind == "cuda" else HOST_FLAGS) + extra).encode())
    for src, text in _with_includes(sources):
        h.update(src.name.encode())
        h.update(text.encode())
    return h.hexdigest()[:16]


def library_path(name: str) -> Path:
    return build_dir() / f"libmstar_{name}-{library_hash(name)}.so"


def _existing(name: str) -> Path | None:
    """A built library with the right hash, in any of the known folders."""
    fname = f"libmstar_{name}-{library_hash(name)}.so"
    folders = [CSRC / "_build", Path(tempfile.gettempdir()) / f"mstar_b200_build_{os.getuid()}"]
    if os.environ.get("MSTAR_BUILD_DIR"):
        folders.insert(0, Path(os.environ["MSTAR_BUILD_DIR"]))
    for d in folders:
        p = d / fname
        if p.is_file():
            return p
    return None


def build_library(name: str, *, force: bool = False) -> Path:
    """Return the path of the built library ``name``, compiling it if needed."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown library {name!r} (known: {sorted(LIBRARIES)})")
    with _lock:
        if not force:
            found = _existing(name)
            if found is not None:
                return found
        kind, sources, extra = LIBRARIES[name]
        out = library_path(name)
        tmp = out.with_suffix(f".tmp{os.getpid()}.so")
        srcs = [str(CSRC / s) for s in sources]
        if kind == "cuda":
            cmd = [find_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), *extra, "-o", str(tmp), *srcs]
            what = f"compiling CUDA library '{name}' for sm_100a"
        else:
            cmd = [shutil.which("g++") or "g++", *HOST_FLAGS, "-I", str(CSRC), *extra,
                   "-o", str(tmp), *srcs]
            what = f"compiling host library '{name}'"
        _log(what + " ...")
        start = time.time()
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        stop = threading.Event()

        def heartbeat():
            while not stop.wait(10.0):
                _log(f"  still {what} ({time.time() - start:.0f} s)")

        beat = threading.Thread(target=heartbeat, daemon=True)
        beat.start()
        try:
            output, _ = proc.communicate()
        finally:
            stop.set()
        if proc.returncode != 0:
            try:
                tmp.unlink()
            except OSError:
                pass
            raise BuildError(f"{what} failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
        os.replace(tmp, out)
        for stale in out.parent.glob(f"libmstar_{name}-*.so"):
            if stale != out:
                try:
                    stale.unlink()
                except OSError:
                    pass
        _log(f"  built {out.name} in {time.time() - start:.1f} s")
        return out


def build_all(*, force: bool = False) -> dict:
    """Compile every library (used by the build check; serving compiles lazily)."""
    return {name: build_library(name, force=force) for name in LIBRARIES}
