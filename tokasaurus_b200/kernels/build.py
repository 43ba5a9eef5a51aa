"""Compile the CUDA sources under ``tokasaurus_b200/csrc`` with nvcc for sm_100a and load them
through ctypes.

Every kernel file exposes plain ``extern "C"`` launchers that take device pointers, sizes and a
stream.  A *module* is one shared library made from one source file and a set of ``-D`` constants
(the attention kernels are specialised by head size this way, so a model compiles only what
it needs).  Libraries are cached by a hash of source text, constants and flags, in
``tokasaurus_b200/csrc/_build`` when that folder can be written, else under the system's
temporary folder.  Nothing here needs a GPU: nvcc cross-compiles.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def find_nvcc() -> str:
    for cand in (
        os.environ.get("TKB_NVCC"),
        os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError(
        "nvcc was not found (looked at $TKB_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
        "the engine's CUDA kernels cannot be built and there is no other execution path"
    )


def build_dir() -> Path:
    env = os.environ.get("TKB_BUILD_DIR")
    cands = [Path(env)] if env else []
    cands.append(CSRC / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"tokasaurus_b200_build_{os.getuid()}")
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for compiled kernels among {[str(c) for c in cands]}")


_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _source_closure(src: Path) -> list[Path]:
    """The source file and every file of this folder it includes, directly or not."""
    seen: dict[Path, None] = {}
    todo = [src]
    while todo:
        p = todo.pop()
        if p in seen or not p.is_file():
            continue
        seen[p] = None
        for name in _INCLUDE.findall(p.read_text()):
            todo.append(CSRC / name)
    return sorted(seen)


def module_path(source: str, defines: dict[str, int | str] | None = None, extra_flags: tuple[str, ...] = ()) -> tuple[Path, list[str]]:
    src = CSRC / source
    if not src.is_file():
        raise KernelBuildError(f"kernel source {src} is missing")
    defines = defines or {}
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    h = hashlib.sha256()
    for dep in _source_closure(src):
        h.update(dep.name.encode())
        h.update(dep.read_bytes())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS + dflags + list(extra_flags)).encode())
    tag = "_".join(f"{k.lower().replace('tkb_', '')}{v}" for k, v in sorted(defines.items()))
    name = f"{src.stem}{'_' + tag if tag else ''}_{h.hexdigest()[:12]}.so"
    cmd_tail = ARCH_FLAGS + BASE_FLAGS + dflags + list(extra_flags) + ["-I", str(CSRC), str(src)]
    return build_dir() / name, cmd_tail


def compile_module(source: str, defines: dict[str, int | str] | None = None, extra_flags: tuple[str, ...] = (), verbose: bool = True) -> Path:
    """Compile (if not cached) and return the path of the shared library."""
    out, cmd_tail = module_path(source, defines, extra_flags)
    if out.is_file():
        return out
    nvcc = find_nvcc()
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc] + cmd_tail + ["-o", str(tmp)]
    if verbose:
        print(f"[tokasaurus_b200] compiling {source} {defines or ''} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    # Print a line now and then while nvcc works, so a first call does not look hung.
    while True:
        try:
            output, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[tokasaurus_b200]   still compiling {source} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed for {source} (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    if verbose:
        print(f"[tokasaurus_b200]   built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_module(source: str, defines: dict[str, int | str] | None = None, extra_flags: tuple[str, ...] = ()) -> ctypes.CDLL:
    path, _ = module_path(source, defines, extra_flags)
    key = str(path)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            compile_module(source, defines, extra_flags)
            try:
                lib = ctypes.CDLL(key)
            except OSError as e:
                raise KernelBuildError(f"cannot load compiled kernels {key}: {e}") from e
            _loaded[key] = lib
        return lib
