"""In-tree compilation of the native code, done at first use.

Two kinds of target:

* the host runtime (page pools, cache manager, scheduler, sampler), C++ with
  pybind11, compiled by g++ and importable without a GPU;
* one shared library per CUDA source under ``kernels/``, compiled by nvcc for
  sm_100a only and loaded through ctypes. A model compiles the libraries whose
  kernels it calls, not the rest.

Outputs go to ``_build/`` beside this file (or to ``$STRIDE_B200_BUILD_DIR``, or
to a per-user temporary folder when the tree is read-only). A target is rebuilt
when the hash of its sources and flags changes. While a compile runs, a line is
printed to stderr every few seconds so that a first call does not look hung.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import importlib.machinery
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_DIR = os.path.join(HERE, "kernels")
RUNTIME_DIR = os.path.join(HERE, "runtime")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -fno-gnu-unique: function-local statics of templates (such as "this kernel's attributes are set")
# must belong to one library; as GNU unique symbols they would be shared by every library that
# instantiates the same template, although each library carries its own copy of the kernel.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
              "-Xcompiler", "-fno-gnu-unique"]
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[stride_b200] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    override = os.environ.get("STRIDE_B200_BUILD_DIR")
    candidates = [override] if override else [os.path.join(HERE, "_build")]
    candidates.append(os.path.join(tempfile.gettempdir(), f"stride_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return path
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {candidates}")


def find_nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and os.path.exists(os.path.join(root, "bin", "nvcc")):
            return os.path.join(root, "bin", "nvcc")
    found = shutil.which("nvcc")
    if not found:
        raise BuildError("nvcc was not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                         "the CUDA kernels of stride_b200 cannot be built")
    return found


def find_cxx() -> str:
    """The host compiler: ``$STRIDE_B200_CXX``, else the system's g++ (a wrapper
    named by ``$CXX`` may link libstdc++ statically, which breaks exceptions and
    streams in a module loaded beside torch), else ``$CXX``."""
    for candidate in (os.environ.get("STRIDE_B200_CXX"), shutil.which("g++"), shutil.which("c++"), os.environ.get("CXX")):
        if candidate:
            return candidate
    raise BuildError("no C++ compiler found (g++, c++ or $CXX)")


def _digest(paths: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _run(cmd: list[str], what: str) -> None:
    done = threading.Event()

    def heartbeat():
        start = time.time()
        while not done.wait(8.0):
            _say(f"still compiling {what} ({time.time() - start:.0f} s)")

    _say(f"compiling {what}")
    t = threading.Thread(target=heartbeat, daemon=True)
    t.start()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True)
    finally:
        done.set()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def _build(target: str, sources: list[str], deps: list[str], make_cmd) -> str:
    """Returns the path of an up-to-date shared object for ``target``."""
    out_dir = build_dir()
    # the tag must not depend on where the tree lies, or a library built in one checkout is built again in a copy of it
    tag = _digest(sources + deps, [a.replace(HERE, "<csrc>") for a in make_cmd("OUT")])
    out = os.path.join(out_dir, f"{target}.{tag}.so")
    if os.path.exists(out):
        return out
    with open(os.path.join(out_dir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(out):
                return out
            tmp = f"{out}.tmp{os.getpid()}"
            _run(make_cmd(tmp), target)
            os.replace(tmp, out)
            for name in os.listdir(out_dir):  # drop stale builds of the same target
                if name.startswith(target + ".") and name.endswith(".so") and name != os.path.basename(out):
                    try:
                        os.unlink(os.path.join(out_dir, name))
                    except OSError:
                        pass
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


def _headers(folder: str) -> list[str]:
    return [os.path.join(folder, f) for f in os.listdir(folder) if f.endswith((".hpp", ".cuh", ".h"))]


def kernel_sources() -> list[str]:
    return sorted(f[:-3] for f in os.listdir(KERNEL_DIR) if f.endswith(".cu"))


def build_kernel_library(name: str) -> str:
    src = os.path.join(KERNEL_DIR, f"{name}.cu")
    if not os.path.exists(src):
        raise BuildError(f"no kernel source {src}")
    extra = os.environ.get("STRIDE_B200_NVCC_FLAGS", "").split()

    def cmd(out):
        return [find_nvcc(), *NVCC_ARCH, *NVCC_FLAGS, *extra, "-I", KERNEL_DIR, "-o", out, src, "-lcuda"]

    deps = _headers(KERNEL_DIR)
    with open(src) as f:     # a source may include another source (a variant that reuses its kernels)
        for line in f:
            line = line.strip()
            if line.startswith('#include "') and line.split('"')[1].endswith(".cu"):
                deps.append(os.path.join(KERNEL_DIR, line.split('"')[1]))
    return _build(f"kernels_{name}", [src], deps, cmd)


def build_external_library(source: str) -> str:
    """A CUDA source from outside the package (a test's own kernel) compiled with the package's flags and
    its kernel headers on the include path."""
    source = os.path.abspath(source)
    if not os.path.exists(source):
        raise BuildError(f"no kernel source {source}")

    def cmd(out):
        return [find_nvcc(), *NVCC_ARCH, *NVCC_FLAGS, "-I", KERNEL_DIR, "-o", out, source, "-lcuda"]

    name = os.path.splitext(os.path.basename(source))[0]
    return _build(f"external_{name}", [source], _headers(KERNEL_DIR), cmd)


def build_runtime() -> str:
    import pybind11

    src = os.path.join(RUNTIME_DIR, "bindings.cpp")
    suffix_free_includes = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", RUNTIME_DIR]

    def cmd(out):
        return [find_cxx(), *CXX_FLAGS, *suffix_free_includes, "-o", out, src]

    return _build("_runtime", [src], _headers(RUNTIME_DIR), cmd)


_runtime_module = None
_kernel_libs: dict[str, ctypes.CDLL] = {}


def load_runtime():
    """The pybind11 module of the host runtime, built on first use."""
    global _runtime_module
    if _runtime_module is None:
        path = build_runtime()
        loader = importlib.machinery.ExtensionFileLoader("_runtime", path)
        spec = importlib.util.spec_from_loader("_runtime", loader, origin=path)
        module = importlib.util.module_from_spec(spec)
        loader.exec_module(module)
        _runtime_module = module
    return _runtime_module


def load_kernel_library(name: str) -> ctypes.CDLL:
    """The ctypes handle of one kernel library, built on first use."""
    lib = _kernel_libs.get(name)
    if lib is None:
        lib = ctypes.CDLL(build_kernel_library(name))
        _kernel_libs[name] = lib
    return lib


def load_external_library(source: str) -> ctypes.CDLL:
    return ctypes.CDLL(build_external_library(source))


def build_all(verbose: bool = True) -> list[str]:
    """Compiles the runtime and every kernel library; returns the paths."""
    out = [build_runtime()]
    for name in kernel_sources():
        out.append(build_kernel_library(name))
    if verbose:
        for p in out:
            _say(f"built {os.path.relpath(p, HERE)}")
    return out
