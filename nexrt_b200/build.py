"""Ahead-of-time / on-demand nvcc build of ``libnexrt_b200.so`` for sm_100a.

Role of the reference's ``nex_n2_5_pro/kernel_build.py:146-202`` (race-free JIT of one ``.so``
per translation unit under ``build/sm90a``): freshness is the newest mtime of a source, of the
headers it includes (recursively, quoted includes only) and of this file; concurrent ranks
serialise on an ``flock`` in the system temp directory; objects and the library are written to a
``.pid.tmp`` name and published with ``os.replace``; build paths that are symlinks or that escape
the build root are refused.  Differences: translation units are compiled in parallel into
objects and linked into ONE in-tree library (so a snapshot of the source tree carries the
binary), and the only architecture is ``-gencode arch=compute_100a,code=sm_100a``.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import re
import shutil
import subprocess
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Iterable, List

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
# NEXRT_TRACE_BUILD=1 selects the timeline variant of the library: the same sources compiled with -DNEXRT_TRACE
# (every kernel records %globaltimer at its phase boundaries, see csrc/common.cuh) into objects and a library of
# their own, so the product library never carries the instrumentation.
TRACE_BUILD = os.environ.get("NEXRT_TRACE_BUILD", "0") == "1"
BUILD_ROOT = PKG / "build" / ("sm100a_trace" if TRACE_BUILD else "sm100a")
LIB_NAME = "libnexrt_b200_trace.so" if TRACE_BUILD else "libnexrt_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"] + (["-DNEXRT_TRACE"] if TRACE_BUILD else [])
_INCLUDE_RE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def validate_build_path(path: Path, root: Path = BUILD_ROOT) -> Path:
    """Refuse symlinked components and paths that leave the build root."""
    root_res = root.resolve()
    cur = path
    while True:
        if cur.is_symlink():
            raise RuntimeError(f"refusing symlinked build path component: {cur}")
        if cur == cur.parent or cur == root or cur == PKG:
            break
        cur = cur.parent
    res = path.resolve()
    if root_res != res and root_res not in res.parents:
        raise RuntimeError(f"build path {path} escapes {root}")
    return path


def _headers_of(src: Path, seen=None) -> Iterable[Path]:
    seen = seen if seen is not None else set()
    try:
        text = src.read_text(errors="replace")
    except OSError:
        return seen
    for name in _INCLUDE_RE.findall(text):
        h = (src.parent / name).resolve()
        if h.is_file() and h not in seen:
            seen.add(h)
            _headers_of(h, seen)
    return seen


def source_mtime(src: Path) -> float:
    """Newest mtime of the source, every quoted header reachable from it, and this helper."""
    times = [src.stat().st_mtime, Path(__file__).stat().st_mtime]
    times += [h.stat().st_mtime for h in _headers_of(src)]
    return max(times)


def is_fresh(out: Path, src: Path) -> bool:
    return out.is_file() and out.stat().st_mtime >= source_mtime(src)


def _lock_file() -> Path:
    tag = hashlib.sha1(str(PKG).encode()).hexdigest()[:12]
    return Path(tempfile.gettempdir()) / f"nexrt_b200_build_{tag}.lock"


def _run(cmd: List[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def compile_object(src: Path, verbose_ptxas: bool = False) -> Path:
    obj = validate_build_path(BUILD_ROOT / (src.stem + ".o"))
    if is_fresh(obj, src):
        return obj
    tmp = obj.with_name(f"{obj.name}.{os.getpid()}.tmp")
    cmd = [nvcc_path(), *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(tmp)]
    if verbose_ptxas:
        cmd += ["-Xptxas", "-v"]
    try:
        _run(cmd)
        os.replace(tmp, obj)
    finally:
        if tmp.exists():
            tmp.unlink()
    return obj


def library_path() -> Path:
    return PKG / LIB_NAME


def build_library(force: bool = False, jobs: int = 0) -> Path:
    """Compile every ``csrc/*.cu`` that is stale and link the in-tree shared library."""
    lib = library_path()
    srcs = sources()
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    if not force and lib.is_file() and all(lib.stat().st_mtime >= source_mtime(s) for s in srcs):
        return lib
    BUILD_ROOT.mkdir(parents=True, exist_ok=True)
    validate_build_path(BUILD_ROOT)
    with open(_lock_file(), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and lib.is_file() and all(lib.stat().st_mtime >= source_mtime(s) for s in srcs):
                return lib  # another rank built it while we waited
            if force:
                for s in srcs:
                    o = BUILD_ROOT / (s.stem + ".o")
                    if o.exists():
                        o.unlink()
            jobs = jobs or min(len(srcs), os.cpu_count() or 4)
            with ThreadPoolExecutor(max_workers=jobs) as pool:
                objs = list(pool.map(compile_object, srcs))
            tmp = lib.with_name(f"{lib.name}.{os.getpid()}.tmp")
            try:
                _run([nvcc_path(), *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), "-lcuda"])
                os.replace(tmp, lib)
            finally:
                if tmp.exists():
                    tmp.unlink()
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


def main(argv=None) -> int:
    """``python -m nexrt_b200.build [--force]``: build (or reuse) the library and print its path."""
    import sys

    args = sys.argv[1:] if argv is None else list(argv)
    print(build_library(force="--force" in args))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
