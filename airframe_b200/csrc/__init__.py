"""Build and load the sm_100a kernel library.

The sources beside this file are compiled with ``nvcc`` into one shared
object, ``_build/libairframe_b200.so``, and loaded with ``ctypes``.  The
build happens at the first call that needs it and again whenever a source
changed (a digest of the sources is kept beside the object).  There is no
other implementation to fall back on: if ``nvcc`` is missing or the build
fails, :class:`KernelLibraryError` is raised.
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
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

SOURCE_DIR = Path(__file__).resolve().parent
LIB_NAME = "libairframe_b200.so"
CHECKED_LIB_NAME = "libairframe_b200_checked.so"
_checked = False


def use_checked_build() -> None:
    """Load the checked build instead (compiled with ``-DAF_BOUNDS_CHECK``: the
    indices that kernels take from data are checked, a bad one is recorded and
    its access skipped; ``kernels.bounds_failures()`` reads the record).  Must
    be called before the library is first used; meant for test runs."""
    global _checked
    if _lib is not None and not _checked:
        raise KernelLibraryError("the kernel library is loaded already; choose the checked build before its first use")
    _checked = True

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


class KernelLibraryError(RuntimeError):
    """The kernel library could not be built or loaded."""


def _say(msg: str) -> None:
    print(f"[airframe_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> list[Path]:
    return sorted(SOURCE_DIR.glob("*.cu"))


def _digest(extra: str = "") -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    for p in sorted(list(SOURCE_DIR.glob("*.cu")) + list(SOURCE_DIR.glob("*.cuh")) + list(SOURCE_DIR.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise KernelLibraryError("nvcc not found: the CUDA kernels cannot be built (set NVCC or PATH)")


def build_dir() -> Path:
    """Where the object lives: ``_build`` beside the sources, or, when that
    place cannot be written, a per-user folder under the temporary directory."""
    override = os.environ.get("AIRFRAME_B200_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    d = SOURCE_DIR / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"airframe_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _run(cmd: list[str], what: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelLibraryError(f"{what} failed ({proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}")


def build(force: bool = False, verbose: bool = True, checked: bool = False) -> Path:
    """Compile every ``.cu`` here for sm_100a and link the shared object.
    Returns its path.  Does nothing when the object is up to date.
    ``checked``: the variant with ``-DAF_BOUNDS_CHECK`` (a library of its own)."""
    out_dir = build_dir()
    name = CHECKED_LIB_NAME if checked else LIB_NAME
    flags = NVCC_FLAGS + (["-DAF_BOUNDS_CHECK"] if checked else [])
    lib = out_dir / name
    stamp = out_dir / (name + ".sha256")
    digest = _digest(" ".join(flags))
    if not force and lib.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return lib
    nvcc = _nvcc()
    srcs = sources()
    if verbose:
        _say(f"building {name} from {len(srcs)} sources for sm_100a in {out_dir}")
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        objs = [out_dir / (s.stem + (".checked.o" if checked else ".o")) for s in srcs]

        def one(pair):
            s, o = pair
            _run([nvcc, *flags, "-I", str(SOURCE_DIR), "-c", str(s), "-o", str(o)], f"compiling {s.name}")
            if verbose:
                _say(f"compiled {s.name} ({time.time() - t0:.0f} s)")

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            list(ex.map(one, zip(srcs, objs)))
        tmp = out_dir / (name + f".tmp{os.getpid()}")
        _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"],
             "linking")
        os.replace(tmp, lib)
        stamp.write_text(digest)
    finally:
        done.set()
    if verbose:
        _say(f"built {lib.name} in {time.time() - t0:.0f} s")
    return lib


_lib = None
_lock = threading.Lock()


def load_library() -> ctypes.CDLL:
    """The loaded kernel library (built first if needed)."""
    global _lib
    with _lock:
        if _lib is None:
            path = build(checked=_checked)
            try:
                _lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelLibraryError(f"cannot load {path}: {e}") from e
            _lib.af_last_error.restype = ctypes.c_char_p
        return _lib
