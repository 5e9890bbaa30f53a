"""Builds the CUDA sources of mashbox_b200/csrc into shared libraries for sm_100a and loads them with ctypes.

Each .cu file becomes one library, compiled with nvcc the first time something needs it (a float32 run never compiles
the bf16 tensor-core kernels) and found again afterwards by a hash of its sources and flags.  Libraries live in
csrc/_build/ inside the package when that folder can be written, else in a per-user folder under the system's
temporary directory; no home directory and no network is needed.  While nvcc runs, a line is printed to stderr every
few seconds.  A missing compiler or a failed build raises KernelError: there is no fallback.
"""
import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

from ..errors import KernelError

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
HEADERS = ["common.cuh", "attention_common.cuh", "tcgen05.cuh"]
LIBRARIES = {            # library name -> (source file, extra compiler flags)
    "elementwise": ("elementwise.cu", []),
    "gemm_f32": ("gemm_f32.cu", []),
    "gemm_tc5": ("gemm_tc5.cu", []),
    "gemm_stream": ("gemm_stream.cu", []),
    "gemv": ("gemv.cu", []),
    "attention_simple": ("attention_simple.cu", []),
    "attention_mma": ("attention_mma.cu", []),                         # head sizes 16, 32, 64, 128
    "attention_mma_wide": ("attention_mma.cu", ["-DMB_ATTN_WIDE"]),    # the other multiples of 16 up to 256
    "attention_tma": ("attention_tma.cu", []),
    "attention_tc5": ("attention_tc5.cu", []),
    "sampling": ("sampling.cu", []),
    "sampling_noalloc": ("sampling_noalloc.cu", []),
    "trace": ("trace.cu", []),
}
EXTRA_SOURCES = {"sampling_noalloc": ["sampling.cu", "sampling_noalloc.h"]}      # files a library includes
_loaded = {}
_lock = threading.Lock()


def find_nvcc():
    for c in (os.environ.get("MASHBOX_NVCC"), shutil.which("nvcc"),
              os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelError("nvcc was not found (looked at MASHBOX_NVCC, PATH, CUDA_HOME and /usr/local/cuda): the CUDA "
                      "kernels of mashbox_b200 cannot be built")


_build_dir = {"path": os.environ.get("MASHBOX_B200_BUILD_DIR")}


def set_build_dir(path):
    """Compiled libraries go to (and are looked for in) this folder from now on."""
    _build_dir["path"] = path


def build_dir():
    if _build_dir["path"]:
        os.makedirs(_build_dir["path"], exist_ok=True)
        return _build_dir["path"]
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}.{threading.get_ident()}")
        open(probe, "w").close()
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"mashbox_b200-build-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _digest(name):
    src, extra = LIBRARIES[name]
    h = hashlib.sha256()
    for f in [src] + HEADERS + EXTRA_SOURCES.get(name, []):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + FLAGS + extra).encode())
    return h.hexdigest()[:16]


def library_path(name):
    return os.path.join(build_dir(), f"libmashbox_b200_{name}-{_digest(name)}.so")


def compile_library(name, verbose=True):
    """Compiles one library if its file is not there yet.  -> path"""
    if name not in LIBRARIES:
        raise KernelError(f"no kernel library named {name}")
    path = library_path(name)
    if os.path.isfile(path):
        return path
    nvcc = find_nvcc()
    src, extra = LIBRARIES[name]
    lock_path = path + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(path):
                return path
            tmp = f"{path}.{os.getpid()}.tmp"
            cmd = [nvcc] + ARCH_FLAGS + FLAGS + extra + ["-I", CSRC, "-o", tmp, os.path.join(CSRC, src)]
            t0 = time.time()
            if verbose:
                print(f"mashbox_b200: compiling {src} for sm_100a ...", file=sys.stderr, flush=True)
            env = dict(os.environ)
            env.setdefault("TMPDIR", tempfile.gettempdir())
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
            while True:
                try:
                    out, _ = proc.communicate(timeout=5)
                    break
                except subprocess.TimeoutExpired:
                    if verbose:
                        print(f"mashbox_b200: still compiling {src} ({time.time() - t0:.0f} s)", file=sys.stderr,
                              flush=True)
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise KernelError(f"nvcc failed on {src}:\n{out[-4000:]}")
            os.replace(tmp, path)
            if verbose:
                print(f"mashbox_b200: built {os.path.basename(path)} in {time.time() - t0:.1f} s", file=sys.stderr,
                      flush=True)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return path


def load_library(name):
    """-> ctypes.CDLL of the named library, compiling it on first use."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def prune():
    """Removes libraries in the build folder that no current source hashes to (left by earlier versions of a file)."""
    d = build_dir()
    current = {os.path.basename(library_path(n)) for n in LIBRARIES}
    for f in os.listdir(d):
        stale_lock = f.endswith(".so.lock") and f[:-5] not in current
        if f.startswith("libmashbox_b200_") and ((f.endswith(".so") and f not in current) or stale_lock):
            try:
                os.remove(os.path.join(d, f))
            except OSError:
                pass


def build_all(verbose=True):
    """Compiles every library (in parallel).  -> {name: path}"""
    out, errors, threads = {}, [], []

    def one(n):
        try:
            out[n] = compile_library(n, verbose)
        except Exception as e:       # collected and raised below
            errors.append(e)
    for n in LIBRARIES:
        th = threading.Thread(target=one, args=(n,))
        th.start()
        threads.append(th)
    for th in threads:
        th.join()
    if errors:
        raise errors[0]
    return out
