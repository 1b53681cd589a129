"""Builds the native libraries in-tree.

Two shared objects are produced next to this file (under ``lib/``):

* ``libllmc_b200.so``  every CUDA kernel of the framework, compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``).  The kernels export plain C entry points that take
  raw device pointers and a CUDA stream, so Python reaches them through ctypes and no PyTorch
  headers are needed at build time (a full rebuild takes seconds, cross-compiles without a GPU).
* ``libllmc_host.so``  the C++ host runtime (data loader, RNG, tokenizer, schedulers, checkpoint IO ...).
* ``libllmc_b200_debug.so``  (``build(debug=True)`` / ``python -m llmc_b200.build --debug``) the kernels with their debug checks on.

A content hash of the sources is stored beside each library; ``build()`` is a no-op when it matches,
so a tree whose libraries were built elsewhere is used as is.
"""
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-ffp-contract=off"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources(sub, exts):
    d = os.path.join(CSRC, sub) if sub else CSRC
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(exts))


def _hash(files, extra):
    h = hashlib.sha256()
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(repr(extra).encode())
    return h.hexdigest()


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), r.stdout))
    return r.stdout


def _build_lib(name, sources, headers, compile_cmd, link_cmd, flags, verbose):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    lib = os.path.join(LIBDIR, name)
    stamp = lib + ".hash"
    digest = _hash(sources + headers, flags)
    if os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
        return lib
    objs = []

    def compile_one(src):
        obj = os.path.join(OBJDIR, name + "." + os.path.basename(src) + ".o")
        out = _run(compile_cmd + flags + ["-I", CSRC, "-c", src, "-o", obj])
        if verbose and out.strip():
            print(out)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(sources)))) as ex:
        objs = list(ex.map(compile_one, sources))
    _run(link_cmd + objs + ["-o", lib])
    with open(stamp, "w") as fh:
        fh.write(digest)
    if verbose:
        print("built", lib)
    return lib


def build_cuda(verbose=False):
    nvcc = _nvcc()
    srcs = _sources("", (".cu",))
    hdrs = _sources("", (".cuh", ".h"))
    return _build_lib("libllmc_b200.so", srcs, hdrs, [nvcc], [nvcc, "-shared", "-Xcompiler", "-fPIC"], NVCC_FLAGS, verbose)


def build_cuda_debug(verbose=False):
    """The same kernels with -DLLMC_DEBUG_CHECKS: every 16-byte access checks its alignment and the embedding / classifier
    kernels check their ids; a failed check is recorded in the status word and the access is skipped or clamped (the role that
    compute-sanitizer runs play for the reference).  Relocatable device code, so that all files share one status pointer.
    Selected at run time with LLMC_DEBUG_CHECKS=1."""
    nvcc = _nvcc()
    srcs = _sources("", (".cu",))
    hdrs = _sources("", (".cuh", ".h"))
    flags = NVCC_FLAGS + ["-rdc=true", "-DLLMC_DEBUG_CHECKS=1"]
    return _build_lib("libllmc_b200_debug.so", srcs, hdrs, [nvcc], [nvcc, "-shared", "-rdc=true", "-gencode", "arch=compute_100a,code=sm_100a",
                                                                    "-Xcompiler", "-fPIC"], flags, verbose)


def build_host(verbose=False):
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    srcs = _sources("host", (".cpp",))
    hdrs = _sources("host", (".h", ".hpp"))
    return _build_lib("libllmc_host.so", srcs, hdrs, [cxx], [cxx, "-shared", "-pthread"], CXX_FLAGS, verbose)


def build(verbose=False, debug=False):
    out = (build_cuda(verbose), build_host(verbose))
    if debug:
        out += (build_cuda_debug(verbose),)
    return out


if __name__ == "__main__":
    build(verbose="-q" not in sys.argv, debug="--debug" in sys.argv)
