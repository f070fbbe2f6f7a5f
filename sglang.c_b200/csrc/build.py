"""Builds the CUDA sources of this folder for sm_100a, one shared library per
.cu file, on first use, and loads them with ctypes.

A library is rebuilt when its source, a header of this folder or the flags change (a hash
is stored beside it).  Libraries are kept in-tree under `csrc/_build/`; if that
folder cannot be written they go to a per-user folder under the system's
temporary directory.  While nvcc runs, a line is printed to stderr every few
seconds, so that a first call that has to compile does not look hung.
"""
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

from .. import log

_HERE = os.path.dirname(os.path.abspath(__file__))
# no fast-math: the 32-bit path relies on IEEE division, sqrt and expf
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]

_lock = threading.RLock()
_loaded = {}
_bounds_check = False


def set_bounds_check(on):
    """From now on load the bounds-check build of every kernel library (compiled with
    -DSGLC_BOUNDS_CHECK into files of their own): indices that kernels take from device memory
    are compared with their ranges before use, see common.cuh.  For tests and for hunting a bad
    index where no memory checker can be run; the ordinary build is what serves."""
    global _bounds_check
    with _lock:
        _bounds_check = bool(on)


def _flags():
    return NVCC_FLAGS + (["-DSGLC_BOUNDS_CHECK"] if _bounds_check else [])


class BuildError(RuntimeError):
    pass


def sources():
    return sorted(f[:-3] for f in os.listdir(_HERE) if f.endswith(".cu"))


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels of this engine cannot be built")


_dir = None


def _build_dir():
    """csrc/_build if it can be written, else a per-user folder under the
    temporary directory; decided once per process."""
    global _dir
    with _lock:
        if _dir is None:
            d = os.path.join(_HERE, "_build")
            try:
                os.makedirs(d, exist_ok=True)
                fd, probe = tempfile.mkstemp(dir=d)
                os.close(fd)
                os.remove(probe)
            except OSError:
                d = os.path.join(tempfile.gettempdir(), f"sglc_b200_build_{os.getuid()}")
                os.makedirs(d, exist_ok=True)
            _dir = d
        return _dir


def _digest(name):
    h = hashlib.sha256()
    h.update(" ".join(_flags()).encode())
    files = [fn for fn in os.listdir(_HERE) if fn == name + ".cu" or fn.endswith((".cuh", ".h"))]
    host = os.path.join(_HERE, "host")              # the host engine's headers
    if os.path.isdir(host):
        files += [os.path.join("host", fn) for fn in os.listdir(host) if fn.endswith(".hpp")]
    for fn in sorted(files):
        with open(os.path.join(_HERE, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    return h.hexdigest()


def lib_path(name):
    return os.path.join(_build_dir(), f"libsglc_{name}{'_chk' if _bounds_check else ''}.so")


def build(name, verbose=False):
    """Compile csrc/<name>.cu if its library is missing or stale; return the path."""
    src = os.path.join(_HERE, name + ".cu")
    if not os.path.exists(src):
        raise BuildError(f"no CUDA source {src}")
    out = lib_path(name)
    stamp = out + ".hash"
    want = _digest(name)
    if os.path.exists(out) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return out
    tmp = out + f".tmp{os.getpid()}_{threading.get_ident()}"
    cmd = [_nvcc()] + _flags() + ["-I", _HERE, "-o", tmp, src]
    t0 = time.time()
    log.info(f"compiling {name}.cu for sm_100a ...", always=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            cwd=os.path.dirname(out))
    while True:
        try:
            out_text, _ = proc.communicate(timeout=5)
            break
        except subprocess.TimeoutExpired:
            log.info(f"... still compiling {name}.cu ({time.time() - t0:.0f} s)", always=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed on {name}.cu:\n{out_text}")
    os.replace(tmp, out)
    with open(stamp, "w") as f:
        f.write(want)
    log.info(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s", always=True)
    if verbose and out_text.strip():
        log.info(out_text, always=True)
    return out


def build_all(names=None, jobs=None):
    """Compile every source (or the named ones), several at a time."""
    names = list(names) if names is not None else sources()
    jobs = jobs or min(len(names), os.cpu_count() or 1) or 1
    errors = []

    def work(n):
        try:
            build(n)
        except Exception as e:  # collected and raised below
            errors.append(e)

    threads = []
    pending = list(names)
    while pending or threads:
        while pending and len(threads) < jobs:
            t = threading.Thread(target=work, args=(pending.pop(0),))
            t.start()
            threads.append(t)
        threads[0].join()
        threads.pop(0)
    if errors:
        raise errors[0]
    return [lib_path(n) for n in names]


def build_app(name="sglc"):
    """Compile csrc/apps/<name>.c, a C program on the engine's C interface, against the host
    engine's library (built first) and return the executable's path (beside the libraries)."""
    build("host_engine")
    src = os.path.join(_HERE, "apps", name + ".c")
    out = os.path.join(_build_dir(), name)
    stamp = out + ".hash"
    h = hashlib.sha256()
    for fn in (src, os.path.join(_HERE, "sglc_engine.h")):
        with open(fn, "rb") as f:
            h.update(f.read())
    want = h.hexdigest()
    if os.path.exists(out) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == want:
                return out
    cc = os.environ.get("CC") or shutil.which("cc") or shutil.which("gcc")
    if not cc:
        raise BuildError("no C compiler found (looked at $CC, cc and gcc)")
    tmp = out + f".tmp{os.getpid()}"
    cmd = [cc, "-std=c11", "-O2", "-D_POSIX_C_SOURCE=200809L", "-I", _HERE, src, "-o", tmp, "-L", _build_dir(),
           "-lsglc_host_engine", "-Wl,-rpath," + _build_dir()]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{cc} failed on apps/{name}.c:\n{proc.stdout}")
    os.replace(tmp, out)
    with open(stamp, "w") as f:
        f.write(want)
    return out


def load(name):
    """The ctypes handle of csrc/<name>.cu's library, built first if needed."""
    with _lock:
        key = (name, _bounds_check)
        lib = _loaded.get(key)
        if lib is None:
            path = build(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
            lib.sglc_error_string.restype = ctypes.c_char_p
            lib.sglc_error_string.argtypes = [ctypes.c_int]
            _loaded[key] = lib
        return lib
