"""Compiles the native code of the package at first use.

Two kinds of libraries, both kept beside the sources (``_lib/`` inside the
package; a per-user folder under the system's temporary directory when the
package folder cannot be written):

* ``_host``: the C++20 host runtime (requests, cache manager, scheduler, step
  packing) as a pybind11 module, built with g++ alone;
* kernel libraries: hand-written CUDA for sm_100a with a C interface, built
  with nvcc and loaded with ctypes: ``core`` (everything that does not depend
  on the head size) and one ``attention_hd<N>`` per head size a model uses, so
  that a first call compiles what its model needs and nothing else.

A library is rebuilt when the hash of its sources and flags changes.  While
compiling, a line goes to stderr for every finished file.  There is no
fallback: when a library cannot be built or loaded the caller gets the
compiler's message.

The reference builds one torch CUDAExtension for sm_86/89/90 at install time
(setup.py:29-74); here nothing is installed and the only target is sm_100a.
"""
from __future__ import annotations

import concurrent.futures
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

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-Wall", "-Wextra", "-fvisibility=hidden"]

HOST_SOURCES = ["host/block_manager.cpp", "host/scheduler.cpp", "host/step_pack.cpp", "host/bindings.cpp"]
CORE_KERNEL_SOURCES = ["kernels/elementwise.cu", "kernels/norm.cu", "kernels/rope_kv.cu",
                       "kernels/gemm_f32.cu", "kernels/sampling.cu", "kernels/gemm_skinny.cu", "kernels/gemm_tc.cu"
                       ]
ATTENTION_SOURCES = ["kernels/attention_generic.cu", "kernels/attention_mma.cu", "kernels/attention_tc.cu"]

_lock = threading.Lock()
_loaded: dict[str, object] = {}


class BuildError(RuntimeError):
    pass


def _say(text: str) -> None:
    sys.stderr.write(f"[lyapunov_engine_b200] {text}\n")
    sys.stderr.flush()


def lib_dir() -> str:
    """Where built libraries live: inside the package if it can be written."""
    override = os.environ.get("LYAPUNOV_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(PKG_DIR, "_lib"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"lyapunov_engine_b200-{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError("no writable folder for compiled libraries (tried " + ", ".join(candidates) + ")")


def _find(tool: str, env: str, extra: list[str]) -> str:
    cand = os.environ.get(env) or shutil.which(tool)
    if cand:
        return cand
    for path in extra:
        if os.path.exists(path):
            return path
    raise BuildError(f"{tool} not found (set {env})")


def _nvcc() -> str:
    return _find("nvcc", "NVCC", ["/usr/local/cuda/bin/nvcc"])


def _cxx() -> str:
    return _find("g++", "CXX", ["/usr/bin/g++"])


def existing(sources: list[str]) -> list[str]:
    return [s for s in sources if os.path.exists(os.path.join(CSRC, s))]


def _hash(sources: list[str], flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    deps = set(sources)
    for root in ("kernels", "host"):
        folder = os.path.join(CSRC, root)
        if os.path.isdir(folder):
            for name in sorted(os.listdir(folder)):
                if name.endswith((".cuh", ".hpp", ".h")):
                    deps.add(f"{root}/{name}")
    for rel in sorted(deps):
        h.update(rel.encode())
        with open(os.path.join(CSRC, rel), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd: list[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n$ {' '.join(cmd)}\n{proc.stdout}")


def _compile_all(jobs: list[tuple[list[str], str]], label: str) -> None:
    """Runs compile commands in parallel and prints a line as each finishes."""
    t0 = time.time()
    workers = max(1, min(len(jobs), os.cpu_count() or 1))
    _say(f"compiling {label}: {len(jobs)} file(s), first use only")
    done = 0
    with concurrent.futures.ThreadPoolExecutor(workers) as pool:
        futures = {pool.submit(_run, cmd, what): what for cmd, what in jobs}
        pending = set(futures)
        while pending:
            finished, pending = concurrent.futures.wait(
                pending, timeout=15, return_when=concurrent.futures.FIRST_COMPLETED)
            for f in finished:
                f.result()
                done += 1
                _say(f"  {label}: {futures[f]} done ({done}/{len(jobs)}, {time.time() - t0:.0f} s)")
            if not finished:
                _say(f"  {label}: still compiling ({done}/{len(jobs)}, {time.time() - t0:.0f} s)")


def _build(name: str, sources: list[str], compiler_flags: list[str], cuda: bool, out_path: str,
           link_flags: list[str]) -> None:
    obj_dir = os.path.join(os.path.dirname(out_path), "obj", name)
    os.makedirs(obj_dir, exist_ok=True)
    jobs, objs = [], []
    tool = _nvcc() if cuda else _cxx()
    for src in sources:
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        objs.append(obj)
        cmd = [tool, *compiler_flags, "-I", os.path.join(CSRC, "kernels"), "-I", os.path.join(CSRC, "host"),
               "-c", os.path.join(CSRC, src), "-o", obj]
        jobs.append((cmd, os.path.basename(src)))
    _compile_all(jobs, name)
    tmp = out_path + f".tmp{os.getpid()}"
    _run([tool, "-shared", *objs, "-o", tmp, *link_flags], f"{name} (link)")
    os.replace(tmp, out_path)
    shutil.rmtree(obj_dir, ignore_errors=True)


def _up_to_date(path: str, digest: str) -> bool:
    stamp = path + ".hash"
    try:
        with open(stamp) as f:
            return f.read().strip() == digest and os.path.exists(path)
    except OSError:
        return False


def _stamp(path: str, digest: str) -> None:
    with open(path + ".hash", "w") as f:
        f.write(digest)


def host_library_path(build: bool = True) -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    path = os.path.join(lib_dir(), "_host" + suffix)
    import pybind11

    flags = CXX_FLAGS + ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    digest = _hash(HOST_SOURCES, flags)
    if not _up_to_date(path, digest):
        if not build:
            raise BuildError(f"{path} is missing or stale")
        _build("_host", HOST_SOURCES, flags, False, path, [])
        _stamp(path, digest)
    return path


def load_host():
    """The pybind11 module of the host runtime."""
    with _lock:
        if "_host" in _loaded:
            return _loaded["_host"]
        path = host_library_path()
        loader = importlib.machinery.ExtensionFileLoader("_host", path)
        spec = importlib.util.spec_from_loader("_host", loader)
        module = importlib.util.module_from_spec(spec)
        loader.exec_module(module)
        _loaded["_host"] = module
        return module


def kernel_library_path(name: str, sources: list[str], defines: list[str], build: bool = True) -> str:
    path = os.path.join(lib_dir(), f"lyapunov_{name}.so")
    flags = NVCC_ARCH + NVCC_FLAGS + defines
    sources = existing(sources)
    digest = _hash(sources, flags)
    if not _up_to_date(path, digest):
        if not build:
            raise BuildError(f"{path} is missing or stale")
        _build(name, sources, flags, True, path, [])
        _stamp(path, digest)
    return path


def load_kernels(name: str, sources: list[str], defines: list[str]):
    """A kernel library as a ctypes.CDLL."""
    import ctypes

    with _lock:
        if name in _loaded:
            return _loaded[name]
        path = kernel_library_path(name, sources, defines)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from e
        _loaded[name] = lib
        return lib


def load_core():
    return load_kernels("core", CORE_KERNEL_SOURCES, [])


def load_attention(head_dim: int):
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise BuildError(f"attention kernels take head sizes 16..256 in steps of 16, got {head_dim}")
    return load_kernels(f"attention_hd{head_dim}", ATTENTION_SOURCES, [f"-DLE_HEAD_DIM={head_dim}"])


def build_all(head_dims=(16, 32, 64, 128)) -> list[str]:
    """Builds every library (the host module, the core kernels and the
    attention kernels for the given head sizes); returns their paths."""
    paths = [host_library_path()]
    paths.append(kernel_library_path("core", CORE_KERNEL_SOURCES, []))
    for hd in head_dims:
        paths.append(kernel_library_path(f"attention_hd{hd}", ATTENTION_SOURCES, [f"-DLE_HEAD_DIM={hd}"]))
    return paths
