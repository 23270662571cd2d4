"""Compile the CUDA sources under csrc/ for sm_100a and load them.

Each library is one .cu file plus compile-time definitions (the attention kernels
are specialised by head size and storage type), built with nvcc into a shared
object whose name carries a hash of the sources and flags, and loaded with ctypes.
A library is built the first time something asks for it, so a model compiles only
what it needs.  Built files go to `csrc/_build/` inside the package when that folder
can be written, else to a per-user folder under the system temp directory.  While
nvcc runs, a line is printed to stderr every few seconds.
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
from typing import Dict, Mapping, Optional, Sequence

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "--expt-relaxed-constexpr"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for candidate in (os.environ.get("CISR_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise BuildError("nvcc was not found (looked at $CISR_NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                     "the engine has no path that runs without its CUDA kernels")


_build_dir: Optional[Path] = None


def build_dir() -> Path:
    global _build_dir
    if _build_dir is None:
        _build_dir = _find_build_dir()
    return _build_dir


def _find_build_dir() -> Path:
    override = os.environ.get("CISR_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"cisr_b200_build_{os.getuid()}")
    for path in candidates:
        try:
            path.mkdir(parents=True, exist_ok=True)
            probe = path / f".probe_{os.getpid()}_{threading.get_ident()}"
            probe.write_text("")
            probe.unlink()
            return path
        except OSError:
            continue
    raise BuildError("no writable folder for built kernels: tried " + ", ".join(str(c) for c in candidates))


_INCLUDE = re.compile(r'^[ \t]*#[ \t]*include[ \t]*"([^"]+)"', re.MULTILINE)


def source_closure(source: Path) -> list:
    """The source and every file under csrc/ it includes, directly or through another file (a .cu file may include
    headers, a .h, or another .cu file), sorted by name."""
    seen, todo = {}, [source]
    while todo:
        path = todo.pop()
        if path.name in seen or not path.exists():
            continue
        seen[path.name] = path
        for name in _INCLUDE.findall(path.read_text()):
            todo.append(CSRC / name)
    return [seen[name] for name in sorted(seen)]


def _digest(source: Path, defines: Mapping[str, object], extra: Sequence[str]) -> str:
    """Hash of everything a library is made from: its source, every file that source includes, the definitions
    and the flags.  An edit to any of them gives the library another name, so a stale build is never loaded."""
    h = hashlib.sha256()
    h.update(source.name.encode())
    for path in source_closure(source):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(list(extra)).encode())
    h.update(repr(ARCH_FLAGS + BASE_FLAGS).encode())
    return h.hexdigest()[:16]


def _all_defines(defines: Optional[Mapping[str, object]]) -> dict:
    """The caller's defines, plus CISR_TRACE=1 when the environment asks for the kernel timeline build."""
    merged = dict(defines or {})
    if os.environ.get("CISR_TRACE", "0") not in ("", "0"):
        merged["CISR_TRACE"] = 1
    return merged


def library_path(source_name: str, defines: Optional[Mapping[str, object]] = None, extra: Sequence[str] = ()) -> Path:
    defines = _all_defines(defines)
    source = CSRC / source_name
    tag = "_".join(f"{k.lower()}{v}" for k, v in sorted(defines.items()))
    stem = source.stem + (f"_{tag}" if tag else "")
    return build_dir() / f"libcisr_{stem}_{_digest(source, defines, extra)}.so"


def compile_library(source_name: str, defines: Optional[Mapping[str, object]] = None, extra: Sequence[str] = (),
                    verbose: bool = True) -> Path:
    """Build (if not built yet) and return the path of the shared object."""
    defines = _all_defines(defines)
    source = CSRC / source_name
    if not source.exists():
        raise BuildError(f"kernel source {source} is missing")
    target = library_path(source_name, defines, extra)
    if target.exists():
        return target
    nvcc = find_nvcc()
    tmp = target.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc] + ARCH_FLAGS + BASE_FLAGS + [f"-D{k}={v}" for k, v in sorted(defines.items())]
    cmd += [f"-I{CSRC}", str(source), "-o", str(tmp)] + list(extra)
    label = source.stem + ("" if not defines else " (" + ", ".join(f"{k}={v}" for k, v in sorted(defines.items())) + ")")
    if verbose:
        print(f"[cisr_b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    start = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env={**os.environ, "TMPDIR": str(target.parent)})
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            if verbose:
                print(f"[cisr_b200] still compiling {label} ({time.time() - start:.0f} s)", file=sys.stderr, flush=True)

    beat = threading.Thread(target=heartbeat, daemon=True)
    beat.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if tmp.exists():
            tmp.unlink()
        raise BuildError(f"nvcc failed for {label}:\n{' '.join(cmd)}\n{out}")
    os.replace(tmp, target)
    if verbose:
        print(f"[cisr_b200] built {target.name} in {time.time() - start:.1f} s", file=sys.stderr, flush=True)
    _drop_superseded(target)
    return target


def _drop_superseded(target: Path) -> None:
    """Earlier builds of the same source with the same definitions (another digest: an edited source) are never loaded
    again; remove them so the build folder holds one library per kernel.  A process that still has one open keeps it
    (the file lives until it is closed)."""
    stem, _, digest = target.stem.rpartition("_")
    for other in target.parent.glob(f"{stem}_*.so"):
        rest = other.stem[len(stem) + 1:]
        if other != target and len(rest) == len(digest) and all(c in "0123456789abcdef" for c in rest):
            try:
                other.unlink()
            except OSError:
                pass


def load_library(source_name: str, defines: Optional[Mapping[str, object]] = None, extra: Sequence[str] = ()) -> ctypes.CDLL:
    key = repr((source_name, sorted((defines or {}).items()), list(extra)))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(source_name, defines, extra)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as err:
                raise BuildError(f"could not load {path}: {err}") from err
            _loaded[key] = lib
        return lib


def compile_many(jobs: Sequence[tuple], workers: Optional[int] = None) -> None:
    """Build several libraries at once; each job is (source_name, defines, extra)."""
    from concurrent.futures import ThreadPoolExecutor

    jobs = [j for j in jobs if not library_path(*j).exists()]
    if not jobs:
        return
    workers = workers or min(len(jobs), max(1, (os.cpu_count() or 2) - 1), 8)
    with ThreadPoolExecutor(max_workers=workers) as pool:
        for _ in pool.map(lambda j: compile_library(*j), jobs):
            pass
