"""Compiles the native code on first use and loads it with ctypes.

Two kinds of library come out of this folder:

  * the host library (cache manager, scheduler): `host/*.cc` with g++, no CUDA needed;
  * kernel libraries: `kernels/*.cu` with nvcc for sm_100a, one library per source file and
    set of `-D` definitions, so that a model compiles only the variants that it needs
    (for example attention for its own head size).

Built files go to `csrc/_build/` inside the package when that folder can be written, else to
a per-user folder under the system's temporary directory. A library is rebuilt when its
sources, its flags or the compiler change. While a compiler runs, a line is printed to
standard error every few seconds.
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

CSRC = Path(__file__).resolve().parent
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra"]

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[research-2_b200] {msg}", file=sys.stderr, flush=True)


def build_dir() -> Path:
    env = os.environ.get("RESEARCH2_B200_BUILD_DIR")
    candidates = [Path(env)] if env else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"research2_b200_build_{os.getuid()}")
    for cand in candidates:
        try:
            cand.mkdir(parents=True, exist_ok=True)
            probe = cand / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return cand
        except OSError:
            continue
    raise BuildError("no writable folder for built libraries (tried: " + ", ".join(map(str, candidates)) + ")")


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built")


def _digest(paths: list[Path], flags: list[str], compiler: str) -> str:
    h = hashlib.sha256()
    h.update(compiler.encode())
    h.update("\0".join(flags).encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd: list[str], what: str) -> None:
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker() -> None:
        while not done.wait(10.0):
            _say(f"still compiling {what} ({time.time() - start:.0f} s)")

    t = threading.Thread(target=ticker, daemon=True)
    t.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n$ {' '.join(cmd)}\n{out}")
    _say(f"compiled {what} in {time.time() - start:.1f} s")


def _headers(folder: Path) -> list[Path]:
    return sorted(list(folder.glob("*.h")) + list(folder.glob("*.cuh")))


def _build_and_load(key: str, sources: list[Path], deps: list[Path], cmd_prefix: list[str], flags: list[str],
                    link_flags: list[str], compiler: str) -> ctypes.CDLL:
    with _lock:
        if key in _loaded:
            return _loaded[key]
        digest = _digest(sources + deps, flags + link_flags, compiler)
        out = build_dir() / f"{key}.{digest}.so"
        if not out.is_file():
            _say(f"compiling {key} (first use)")
            tmp = out.with_suffix(f".tmp{os.getpid()}.so")
            _run(cmd_prefix + flags + ["-shared", "-o", str(tmp)] + [str(s) for s in sources] + link_flags, key)
            os.replace(tmp, out)
            for stale in out.parent.glob(f"{key}.*.so"):
                if stale != out and ".tmp" not in stale.name:
                    try:
                        stale.unlink()
                    except OSError:
                        pass
        try:
            lib = ctypes.CDLL(str(out))
        except OSError as err:
            raise BuildError(f"loading {out} failed: {err}") from None
        _loaded[key] = lib
        return lib


def host_library() -> ctypes.CDLL:
    """The cache manager and the scheduler (no CUDA)."""
    folder = CSRC / "host"
    sources = sorted(folder.glob("*.cc"))
    gxx = shutil.which("g++") or "g++"
    flags = list(GXX_FLAGS)
    if os.environ.get("R2_HOST_SANITIZE") == "1":
        # for the CPU tests: run python with LD_PRELOAD set to g++'s libasan.so and libubsan.so
        flags = ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined"] + [f for f in flags if f != "-O2"]
    return _build_and_load("r2host", sources, _headers(folder), [gxx], flags, [], gxx)


def kernel_library(source: str, defines: dict[str, int | str] | None = None) -> ctypes.CDLL:
    """One `kernels/<source>.cu` built for sm_100a with the given -D definitions."""
    folder = CSRC / "kernels"
    path = folder / f"{source}.cu"
    if not path.is_file():
        raise BuildError(f"no kernel source {path}")
    defines = defines or {}
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    tag = "_".join(f"{k.lower()}{v}" for k, v in sorted(defines.items()))
    key = f"r2k_{source}" + (f"_{tag}" if tag else "")
    nvcc = find_nvcc()
    flags = NVCC_ARCH + NVCC_FLAGS + dflags + ["-I", str(folder)]
    return _build_and_load(key, [path], _headers(folder), [nvcc], flags, [], nvcc)
