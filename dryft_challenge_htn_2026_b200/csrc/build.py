"""Compiles the .cu files of this folder for sm_100a with nvcc and loads them with ctypes.

Each source becomes one shared object under ``csrc/_build/`` (in the tree, so that a built copy
travels with the folder), named after the source, its compile-time constants and a hash of the
source text and flags. A missing object is compiled on first use, with a progress line on stderr
every few seconds, so a fresh checkout needs nothing but nvcc. There is no fallback: if the
compiler or a CUDA device is missing, loading raises.
"""
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_libs = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc not found (set NVCC or put it on PATH): the CUDA kernels cannot be built, "
                           "and this library has no other way to run")


def _say(msg):
    print(f"[dryft-b200] {msg}", file=sys.stderr, flush=True)


def build_dir():
    """``csrc/_build`` in the tree; if the tree cannot be written (another user's checkout), a
    folder of this user's under the temporary directory."""
    try:
        os.makedirs(BUILD_DIR, exist_ok=True)
        if os.access(BUILD_DIR, os.W_OK):
            return BUILD_DIR
    except OSError:
        pass
    import tempfile
    alt = os.path.join(tempfile.gettempdir(), f"dryft_b200_build_{os.getuid()}")
    os.makedirs(alt, exist_ok=True)
    return alt


def lib_path(source, defines=None):
    defines = dict(defines or {})
    with open(os.path.join(HERE, source), "rb") as f:
        text = f.read()
    for header in sorted(n for n in os.listdir(HERE) if n.endswith((".cuh", ".h"))):
        with open(os.path.join(HERE, header), "rb") as f:
            text += f.read()
    tag = "_".join(f"{k}{v}" for k, v in sorted(defines.items()))
    h = hashlib.sha1(text + repr((ARCH_FLAGS, NVCC_FLAGS, sorted(defines.items()))).encode()).hexdigest()[:12]
    stem = os.path.splitext(source)[0]
    name = f"{stem}{'_' + tag if tag else ''}_{h}.so"
    in_tree = os.path.join(BUILD_DIR, name)
    return in_tree if os.path.exists(in_tree) else os.path.join(build_dir(), name)


def compile_lib(source, defines=None, verbose=False):
    """Builds the shared object for ``source`` if it is not there yet; returns its path."""
    out = lib_path(source, defines)
    if os.path.exists(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *(f"-D{k}={v}" for k, v in sorted((defines or {}).items())),
           *(["-Xptxas", "-v"] if verbose else []), "-I", HERE, "-o", tmp, os.path.join(HERE, source)]
    _say(f"compiling {source} {defines or ''} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"still compiling {source} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=heartbeat, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed for {source}:\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    if verbose:
        print(log)
    return out


def load_lib(source, defines=None):
    """ctypes handle of the (built on demand) shared object of ``source``."""
    key = (source, tuple(sorted((defines or {}).items())))
    with _lock:
        lib = _libs.get(key)
        if lib is None:
            lib = ctypes.CDLL(compile_lib(source, defines))
            _libs[key] = lib
    return lib


def loaded_libs():
    """{(source, defines): handle} of the objects loaded so far."""
    return dict(_libs)


def build_all(head_dims=(16, 32, 64, 128), verbose=False):
    """Compiles every kernel file (attention once per head size), in parallel."""
    from concurrent.futures import ThreadPoolExecutor

    jobs = [("elementwise.cu", None), ("attention_generic.cu", None), ("gemm.cu", None), ("gemv_stream.cu", None),
            ("gemm_tc.cu", None), ("sampling.cu", None),
            ("sample_noalloc.cu", None)]
    jobs += [("attention_bf16.cu", {"HD": hd}) for hd in head_dims]
    jobs += [("attention_tc.cu", {"HD": hd}) for hd in head_dims if hd in (64, 128)]
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        return list(ex.map(lambda j: compile_lib(j[0], j[1], verbose), jobs))
