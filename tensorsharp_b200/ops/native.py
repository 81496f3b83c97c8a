"""Build and load the in-tree CUDA library (``tensorsharp_b200/_native/libtsb200.so``).

The library is plain ``extern "C"``: Python passes raw device pointers and the current
CUDA stream through ctypes, so a kernel launch costs one foreign call and the calls are
capturable in CUDA graphs.  Sources live in ``tensorsharp_b200/csrc`` and are compiled
for ``sm_100a`` only.  On a machine with a GPU a missing library is an error, never a
silent fallback.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional

_PKG = Path(__file__).resolve().parent.parent
CSRC = _PKG / "csrc"
OUT_DIR = _PKG / "_native"
LIB_PATH = OUT_DIR / "libtsb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
# Sources that only a single-GPU call may load (kept out of multi-GPU snapshots).
SINGLE_GPU_ONLY: List[str] = []


class NativeLibraryError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise NativeLibraryError("nvcc not found; cannot build the sm_100a library")


def sources() -> List[Path]:
    return sorted(p for p in CSRC.iterdir() if p.suffix in (".cu", ".cpp"))


def _stamp(src: Path) -> str:
    h = hashlib.sha1()
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, jobs: Optional[int] = None) -> Path:
    """Compile every source under ``csrc`` for sm_100a and link the shared library.
    Objects are cached by content hash, so an unchanged tree is a no-op."""
    OUT_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs, todo = [], []
    for src in sources():
        obj = OUT_DIR / (src.stem + ".o")
        stamp = OUT_DIR / (src.stem + ".stamp")
        objs.append(obj)
        want = _stamp(src)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != want:
            todo.append((src, obj, stamp, want))

    def compile_one(item):
        src, obj, stamp, want = item
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (OUT_DIR / (src.stem + ".ptxas.log")).write_text(r.stderr)
        if r.returncode != 0:
            raise NativeLibraryError(f"nvcc failed for {src.name}:\n{r.stderr[-6000:]}")
        if verbose:
            sys.stderr.write(f"[build] {src.name}\n")
        stamp.write_text(want)

    if todo:
        with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 2)) as ex:
            list(ex.map(compile_one, todo))
    if todo or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-gencode",
               "arch=compute_100a,code=sm_100a", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise NativeLibraryError(f"link failed:\n{r.stderr[-4000:]}")
    return LIB_PATH


def build_tests(force: bool = False) -> List[Path]:
    """Compile the stand-alone C++ test programs under ``csrc/tests`` against the library (``_native/<name>``, found
    next to the library at run time through an ``$ORIGIN`` run path).  They take no Python: ``_native/native_check``."""
    lib_path = build()
    nvcc = _nvcc()
    out: List[Path] = []
    for src in sorted((CSRC / "tests").glob("*.cu")):
        exe = OUT_DIR / src.stem
        stamp = OUT_DIR / (src.stem + ".stamp")
        want = hashlib.sha1(src.read_bytes()).hexdigest()
        if force or not exe.exists() or not stamp.exists() or stamp.read_text() != want or exe.stat().st_mtime < lib_path.stat().st_mtime:
            cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17", str(src), "-o", str(exe),
                   "-L", str(OUT_DIR), "-ltsb200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise NativeLibraryError(f"nvcc failed for tests/{src.name}:\n{r.stderr[-4000:]}")
            stamp.write_text(want)
        out.append(exe)
    return out


def is_stale() -> bool:
    """True when a source or header differs from what the objects were compiled from."""
    for src in sources():
        stamp = OUT_DIR / (src.stem + ".stamp")
        if not stamp.exists() or stamp.read_text() != _stamp(src):
            return True
    return False


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises :class:`NativeLibraryError` if it has not been built."""
    global _lib
    if _lib is None:
        if LIB_PATH.exists() and is_stale():
            build()                      # sources changed since the library was linked
        if not LIB_PATH.exists():
            raise NativeLibraryError(
                f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(or tensorsharp_b200.ops.native.build()) before using the CUDA path")
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.tsb_last_error.restype = ctypes.c_char_p
    return _lib


def available() -> bool:
    return LIB_PATH.exists()


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().tsb_last_error().decode("utf-8", "replace")
        raise NativeLibraryError(f"{what or 'native call'} failed (code {rc}): {msg}")


def main(argv: Optional[List[str]] = None) -> int:
    """``python -m tensorsharp_b200.ops.native [--force] [--tests] [--jobs N] [--quiet]``: build the library (and the
    stand-alone test programs) from the command line, as the reference's ``build-linux.sh --cuda --tests`` does for its
    native bridge.  The target is always sm_100a."""
    import argparse
    ap = argparse.ArgumentParser(description="Build the sm_100a library in place")
    ap.add_argument("--force", action="store_true", help="recompile every source")
    ap.add_argument("--tests", action="store_true", help="also build the stand-alone C++ test programs")
    ap.add_argument("--jobs", type=int, default=None, help="parallel compiler processes (default: min(8, cores))")
    ap.add_argument("--quiet", action="store_true")
    a = ap.parse_args(argv)
    try:
        path = build(force=a.force, verbose=not a.quiet, jobs=a.jobs)
        built = [path] + (build_tests(force=a.force) if a.tests else [])
    except NativeLibraryError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    for b in built:
        print(b)
    return 0


if __name__ == "__main__":
    sys.exit(main())
