"""In-tree build of the native libraries.

Two shared objects are produced next to the sources, under ``parameter_server_b200/lib``:

* ``libpsb_kernels.so`` — every CUDA kernel, compiled for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``), exported through a C ABI and
  loaded with ctypes.  No torch headers are involved, so a full rebuild takes
  seconds and nvcc cross-compiles on a machine without a GPU.
* ``_psb_host*.so`` — the host runtime (control-plane van, executor, parsers,
  slot reader, ...) as a pybind11 module compiled with g++.

Objects are rebuilt only when a source or header is newer than the object.  Beside each library
sits a ``.stamp`` file with a digest of the sources and flags it was built from; a loader that
finds the digest unchanged uses the library as it is (no object files are needed for that, so
a tree copied to another machine with its built libraries does not rebuild), any edit of a
source or header triggers a rebuild on the next load.  Builds take a file lock, so several
processes (one per GPU) starting at once build once.
"""
from __future__ import annotations

import contextlib
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent
CSRC = PKG / "csrc"
HOST = PKG / "csrc" / "host"
LIB = PKG / "lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall", "-Wno-sign-compare"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(src_paths, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(p.stat().st_mtime > t for p in src_paths)


def _run(cmd, log: Path | None = None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)))
    return r


def kernels_lib_path() -> Path:
    return LIB / "libpsb_kernels.so"


def host_lib_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return LIB / ("_psb_host" + suffix)


def _digest(paths, flags) -> str:
    h = hashlib.sha256(" ".join(flags).encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _fresh(out: Path, digest: str) -> bool:
    stamp = out.with_suffix(".stamp")
    try:
        return out.exists() and stamp.read_text().strip() == digest
    except OSError:
        return False


@contextlib.contextmanager
def _build_lock():
    LIB.mkdir(exist_ok=True)
    with open(LIB / ".build.lock", "w") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    extra = os.environ.get("PSB_NVCC_EXTRA", "").split()
    digest = _digest(sources + headers, NVCC_FLAGS + extra)
    out = kernels_lib_path()
    if not force and _fresh(out, digest):
        return out
    with _build_lock():
        if not force and _fresh(out, digest):      # another process built it while this one waited
            return out
        return _build_kernels_locked(sources, headers, digest, force, verbose)


def _build_kernels_locked(sources, headers, digest, force, verbose) -> Path:
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _newer([src] + headers, obj):
            cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("PSB_NVCC_EXTRA", "").split(), "-I", str(CSRC)]
            cmd += ["-c", str(src), "-o", str(obj)]
            jobs.append((cmd, OBJ / (src.stem + ".log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for r in ex.map(lambda j: _run(*j), jobs):
                if verbose:
                    sys.stderr.write(r.stderr)
    objs = [OBJ / (s.stem + ".o") for s in sources]
    out = kernels_lib_path()
    tmp = out.with_suffix(".so.tmp")
    _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart", "-lcuda"])
    os.replace(tmp, out)
    out.with_suffix(".stamp").write_text(digest)
    return out


def build_host(force: bool = False) -> Path | None:
    if not HOST.is_dir():
        return None
    sources = sorted(HOST.glob("*.cc"))
    if not sources:
        return None
    headers = list(HOST.glob("*.h"))
    digest = _digest(sources + headers, CXX_FLAGS + [os.environ.get("PSB_CXX", "g++")])
    out = host_lib_path()
    if not force and _fresh(out, digest):
        return out
    with _build_lock():
        if not force and _fresh(out, digest):
            return out
        return _build_host_locked(sources, headers, digest, force)


def _build_host_locked(sources, headers, digest, force) -> Path:
    import pybind11

    OBJ.mkdir(exist_ok=True)
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(HOST)]
    jobs = []
    for src in sources:
        obj = OBJ / ("host_" + src.stem + ".o")
        if force or _newer([src] + headers, obj):
            jobs.append(([os.environ.get("PSB_CXX", "g++"), *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)], None))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
    objs = [OBJ / ("host_" + s.stem + ".o") for s in sources]
    out = host_lib_path()
    tmp = out.with_suffix(".tmp")
    _run([os.environ.get("PSB_CXX", "g++"), "-shared", "-Wl,-Bsymbolic", "-o", str(tmp), *map(str, objs), "-pthread", "-lz"])
    os.replace(tmp, out)
    out.with_suffix(".stamp").write_text(digest)
    return out


def build_host_selftest(sanitizer: str = "thread") -> Path | None:
    """Compile the native self-test of the host runtime (``csrc/host/selftest``) with a sanitizer
    (``thread`` or ``address,undefined``).  Returns the executable, or None when the compiler or its
    sanitizer runtime is missing."""
    src = HOST / "selftest" / "selftest_main.cpp"
    LIB.mkdir(exist_ok=True)
    out = LIB / ("host_selftest_" + sanitizer.split(",")[0])
    headers = list(HOST.glob("*.h"))
    if not _newer([src] + headers, out):
        return out
    cmd = [os.environ.get("PSB_CXX", "g++"), "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={sanitizer}",
           "-pthread", str(src), "-o", str(out), "-lz"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stderr[-2000:])
        return None
    return out


def build_all(force: bool = False, verbose: bool = False):
    k = build_kernels(force=force, verbose=verbose)
    h = build_host(force=force)
    return k, h


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
