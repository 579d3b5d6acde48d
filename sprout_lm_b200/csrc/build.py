"""Builds the CUDA kernel library for sm_100a with nvcc and caches it beside the sources.

The library is one shared object with a C interface (loaded with ctypes), so a build needs
nvcc only: no Python headers and no framework headers.  The object's name carries a hash of
the sources and flags; a fresh checkout compiles at the first call, prints a line per file
meanwhile, and later calls load the cached object.  The build folder is ``csrc/_build`` when
that can be written, else a per-user folder under the system's temporary directory.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

SOURCE_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    candidates = [shutil.which("nvcc")]
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    for path in candidates:
        if path and os.path.isfile(path) and os.access(path, os.X_OK):
            return path
    raise BuildError("nvcc not found (looked on PATH, in CUDA_HOME and in /usr/local/cuda/bin); "
                     "the kernels cannot be compiled and there is no fallback.")


def sources() -> list[Path]:
    return sorted(SOURCE_DIR.glob("*.cu"))


def extra_flags_from_environment() -> tuple[str, ...]:
    """SPROUT_BUILD_FLAGS adds compiler flags (an instrumented build: ``-DFFN_STAMPS``); the library's
    name carries them, so such a build lives beside the ordinary one."""
    return tuple(os.environ.get("SPROUT_BUILD_FLAGS", "").split())


def _digest(nvcc: str, extra_flags: tuple[str, ...] = ()) -> str:
    h = hashlib.sha256()
    for path in sorted(list(SOURCE_DIR.glob("*.cu")) + list(SOURCE_DIR.glob("*.cuh")) + list(SOURCE_DIR.glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + list(extra_flags)).encode())
    try:
        h.update(subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.encode())
    except OSError:
        pass
    return h.hexdigest()[:16]


def _build_dir() -> Path:
    preferred = SOURCE_DIR / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write_probe_{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"sprout_lm_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _say(message: str, verbose: bool) -> None:
    if verbose:
        print(f"[sprout_lm_b200 build] {message}", file=sys.stderr, flush=True)


def library_path(build: bool = True, verbose: bool = True, extra_flags: tuple[str, ...] = ()) -> Path:
    """Path of the built library, compiling it first if needed (and ``build``)."""
    nvcc = find_nvcc()
    out_dir = _build_dir()
    extra_flags = tuple(extra_flags) + extra_flags_from_environment()
    target = out_dir / f"libsprout_kernels_{_digest(nvcc, extra_flags)}.so"
    if target.exists():
        return target
    if not build:
        raise BuildError(f"{target} has not been built.")
    files = sources()
    started = time.time()
    _say(f"compiling {len(files)} CUDA files for sm_100a into {out_dir} (first call only)", verbose)
    env = dict(os.environ)
    env.setdefault("TMPDIR", str(out_dir))     # nvcc's intermediates: a place this user can write
    objects = []

    def compile_one(path: Path) -> Path:
        obj = out_dir / f"{path.stem}_{os.getpid()}.o"
        cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *extra_flags, "-I", str(SOURCE_DIR), "-c", str(path), "-o", str(obj)]
        t0 = time.time()
        done = subprocess.run(cmd, capture_output=True, text=True, env=env)
        if done.returncode != 0:
            raise BuildError(f"nvcc failed on {path.name}:\n{done.stdout}\n{done.stderr}")
        _say(f"  {path.name} done in {time.time() - t0:.1f}s", verbose)
        if done.stderr.strip() and verbose:
            sys.stderr.write(done.stderr)
        return obj

    workers = max(1, min(len(files), (os.cpu_count() or 2)))
    try:
        with ThreadPoolExecutor(workers) as pool:
            objects = list(pool.map(compile_one, files))
    except BaseException:
        for path in files:                   # a failed build leaves no objects behind
            (out_dir / f"{path.stem}_{os.getpid()}.o").unlink(missing_ok=True)
        raise
    partial = out_dir / f"{target.name}.{os.getpid()}.tmp"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(partial), *map(str, objects)]
    done = subprocess.run(link, capture_output=True, text=True, env=env)
    for obj in objects:
        obj.unlink(missing_ok=True)
    if done.returncode != 0:
        raise BuildError(f"linking failed:\n{done.stdout}\n{done.stderr}")
    os.replace(partial, target)          # atomic: a concurrent builder sees nothing or the whole file
    for stale in out_dir.glob("libsprout_kernels_*.so"):
        if stale != target and not extra_flags:          # an instrumented build leaves the ordinary one alone
            try:
                stale.unlink()               # libraries of older sources
            except OSError:
                pass
    _say(f"built {target.name} in {time.time() - started:.1f}s", verbose)
    return target


if __name__ == "__main__":
    print(library_path())
