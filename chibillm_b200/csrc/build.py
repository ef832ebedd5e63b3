"""Compiles the CUDA sources of this folder for sm_100a into shared libraries.

The libraries export plain C entry points (no Python or torch headers), so a
file compiles in seconds and the result is loaded with ``ctypes``.  A library
is rebuilt when the hash of its sources and flags changes; it is written next
to the package (``chibillm_b200/_lib``) or, when that folder cannot be written,
under the system's temporary folder.  The compile runs at the first call that
needs the library and prints a line per file while it works.
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
from typing import Dict, List, Optional, Sequence

CSRC = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.dirname(CSRC)

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
                "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "static"]

# name of library -> sources (relative to this folder)
LIBRARIES: Dict[str, List[str]] = {
    "chibi_kernels": ["elementwise.cu", "gemm_simt.cu", "gemm_tcgen05.cu", "attention_generic.cu",
                      "sampling.cu"],
    # one library per head size: built with -DCHIBI_HEAD_DIM=<d> when a model needs it
    "chibi_attention_mma": ["attention_mma.cu"],
    # prompt attention on tcgen05, head sizes 64 and 128
    "chibi_attention_tc": ["attention_tcgen05.cu"],
}
TCGEN05_ATTENTION_HEAD_DIMS = (64, 128)
# head sizes whose attention library build_all() makes ahead of time
PREBUILT_HEAD_DIMS = (16, 32, 48, 64, 128)


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[chibillm_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CHIBILLM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at CHIBILLM_NVCC, PATH, CUDA_HOME, /usr/local/cuda); "
                     "the CUDA kernels of chibillm_b200 cannot be compiled")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = tempfile.NamedTemporaryFile(dir=path, delete=True)
        probe.close()
        return True
    except OSError:
        return False


def library_dir() -> str:
    override = os.environ.get("CHIBILLM_LIB_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(PACKAGE, "_lib")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"chibillm_b200-lib-{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} can be written")


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for name in list(sources) + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:12]


def library_path(name: str, defines: Sequence[str] = ()) -> str:
    sources = LIBRARIES[name]
    flags = ARCH_FLAGS + COMMON_FLAGS + [f"-D{d}" for d in defines]
    tag = _digest(sources, flags)
    suffix = ("_" + "_".join(d.replace("=", "") for d in defines)) if defines else ""
    return os.path.join(library_dir(), f"lib{name}{suffix}_{tag}.so")


def _run(cmd: List[str]) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"command failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}")


def ensure_library(name: str, defines: Sequence[str] = (), verbose: bool = True) -> str:
    """Build library ``name`` if its current version is not there; return its path."""
    target = library_path(name, defines)
    if os.path.isfile(target):
        return target
    nvcc = find_nvcc()
    sources = LIBRARIES[name]
    flags = ARCH_FLAGS + COMMON_FLAGS + [f"-D{d}" for d in defines]
    out_dir = os.path.dirname(target)
    work = tempfile.mkdtemp(prefix=f"build-{name}-", dir=out_dir)
    started = time.time()
    try:
        if verbose:
            _say(f"compiling {name} ({len(sources)} files) for sm_100a with {nvcc}")

        def compile_one(src: str) -> str:
            obj = os.path.join(work, os.path.splitext(src)[0] + ".o")
            t0 = time.time()
            _run([nvcc] + flags + ["-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj])
            if verbose:
                _say(f"  {src} done in {time.time() - t0:.1f} s")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            objects = list(pool.map(compile_one, sources))
        tmp_so = os.path.join(work, "out.so")
        _run([nvcc] + ARCH_FLAGS + ["-shared", "-cudart", "static", "-Xcompiler", "-fPIC",
                                    "-o", tmp_so] + objects)
        os.replace(tmp_so, target)
        if verbose:
            _say(f"{os.path.basename(target)} ready in {time.time() - started:.1f} s")
    finally:
        shutil.rmtree(work, ignore_errors=True)
    # older versions of the same library are of no use any more
    prefix = f"lib{name}" + (("_" + "_".join(d.replace("=", "") for d in defines)) if defines else "") + "_"
    for f in os.listdir(out_dir):
        full = os.path.join(out_dir, f)
        if f.startswith(prefix) and f.endswith(".so") and full != target:
            rest = f[len(prefix):-3]
            if len(rest) == 12 and all(c in "0123456789abcdef" for c in rest):
                try:
                    os.remove(full)
                except OSError:
                    pass
    return target


# ------------------------------------------------------------------ the host-side runtime
HOST_SOURCES = ["runtime.cc"]
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-static-libstdc++", "-static-libgcc"]


def find_cxx() -> str:
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++", "/usr/bin/g++", "/opt/gcc/bin/g++",
                 "/usr/local/bin/g++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    raise BuildError("no C++ compiler was found (looked at CXX, g++, c++, clang++); the host-side runtime "
                     "of chibillm_b200 (cache manager, scheduler) cannot be compiled")


def _host_library(stem: str, sources: Sequence[str], what: str, verbose: bool) -> str:
    """A library of plain C++ (no CUDA), built with the host compiler when its current version is absent."""
    h = hashlib.sha256()
    for name in sources:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(HOST_FLAGS).encode())
    target = os.path.join(library_dir(), f"lib{stem}_{h.hexdigest()[:12]}.so")
    if os.path.isfile(target):
        return target
    cxx = find_cxx()
    started = time.time()
    fd, tmp = tempfile.mkstemp(suffix=".so", dir=os.path.dirname(target))
    os.close(fd)
    try:
        _run([cxx] + HOST_FLAGS + [os.path.join(CSRC, s) for s in sources] + ["-o", tmp])
        os.chmod(tmp, 0o755)
        os.replace(tmp, target)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)
    if verbose:
        _say(f"{os.path.basename(target)} ({what}, {cxx}) ready in {time.time() - started:.1f} s")
    for f in os.listdir(os.path.dirname(target)):
        full = os.path.join(os.path.dirname(target), f)
        if f.startswith(f"lib{stem}_") and f.endswith(".so") and full != target:
            try:
                os.remove(full)
            except OSError:
                pass
    return target


def runtime_library(verbose: bool = True) -> str:
    """The cache manager, the scheduler and the batch packing: plain C++, no CUDA."""
    return _host_library("chibi_runtime", HOST_SOURCES, "host runtime", verbose)


def reference_library(verbose: bool = True) -> str:
    """Plain C++ restatements of the device operations (reference_ops.cc): what the tests compare
    every kernel with.  Nothing on the path of generation loads it."""
    return _host_library("chibi_reference", ["reference_ops.cc"], "plain C++ reference of the kernels", verbose)


def attention_library(head_dim: int, verbose: bool = True) -> str:
    return ensure_library("chibi_attention_mma", (f"CHIBI_HEAD_DIM={head_dim}",), verbose)


def attention_tc_library(head_dim: int, verbose: bool = True) -> str:
    return ensure_library("chibi_attention_tc", (f"CHIBI_HEAD_DIM={head_dim}",), verbose)


def prepare(head_dims: Sequence[int] = (), bfloat16: bool = True, verbose: bool = True) -> None:
    """Builds side by side what a model with these head sizes will load and is not there yet: the
    kernel library, the host runtime and, for bfloat16, the attention libraries of each head size
    that the tensor-core kernels take.  Loading them one after the other, each built when first
    asked for, took 17 s from a fresh checkout; together they take as long as the slowest."""
    jobs = [lambda: runtime_library(verbose), lambda: ensure_library("chibi_kernels", verbose=verbose)]
    if bfloat16:
        for d in sorted(set(int(d) for d in head_dims)):
            if d % 16 == 0 and 0 < d <= 256:
                jobs.append(lambda d=d: attention_library(d, verbose))
            if d in TCGEN05_ATTENTION_HEAD_DIMS:
                jobs.append(lambda d=d: attention_tc_library(d, verbose))
    with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
        for done in [pool.submit(job) for job in jobs]:
            done.result()


def build_all(verbose: bool = True) -> List[str]:
    out = [runtime_library(verbose), reference_library(verbose), ensure_library("chibi_kernels", verbose=verbose)]
    with ThreadPoolExecutor(max_workers=4) as pool:
        out += list(pool.map(lambda d: attention_library(d, verbose), PREBUILT_HEAD_DIMS))
        out += list(pool.map(lambda d: attention_tc_library(d, verbose), TCGEN05_ATTENTION_HEAD_DIMS))
    return out


if __name__ == "__main__":
    for p in build_all():
        print(p)
