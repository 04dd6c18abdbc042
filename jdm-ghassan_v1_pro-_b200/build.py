"""In-tree native build: two shared objects next to this file.

* ``_gb200_host.so``  - C++20 host runtime (RNG, dtype codecs, shard I/O, data loader,
  tokenizer, checkpoint / GGUF / GAI codecs, quantisers, sampler) bound with pybind11.
  Needs only g++; importable on machines without a GPU.
* ``_gb200_cuda.so``  - every sm_100a kernel, compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a`` and exported as ``extern "C"``
  launchers that take raw device pointers and a ``cudaStream_t``.  Loaded with
  ``ctypes`` (no torch headers are needed to compile it, so a rebuild takes seconds).

Objects are cached under ``build/`` and recompiled when a source or header is newer.
Run ``python -m ghassan_b200.build`` or call :func:`build_all`.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
HOST_SO = os.path.join(HERE, "_gb200_host.so")
CUDA_SO = os.path.join(HERE, "_gb200_cuda.so")

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-Xptxas", "-v", "-DNDEBUG",
]
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function",
             "-pthread"]


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def _headers(sub):
    out = []
    for root, _, files in os.walk(os.path.join(CSRC, sub)):
        for f in files:
            if f.endswith((".h", ".hpp", ".cuh")):
                out.append(os.path.join(root, f))
    return out


def _run(cmd, log_path=None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + p.stdout)
    if p.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + p.stdout[-6000:])
    return p.stdout


def _link(cmd, target, inputs):
    """Link to a temporary name and rename: a reader (an import in another process, a copy of the tree) sees the old
    library or the new one, never a half-written file."""
    tmp = target + ".tmp%d" % os.getpid()
    try:
        _run(cmd + ["-o", tmp] + inputs)
        os.replace(tmp, target)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)


def _sources(sub, ext):
    d = os.path.join(CSRC, sub)
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(ext))


def build_host(verbose=False, force=False):
    import pybind11
    os.makedirs(os.path.join(BUILD, "host"), exist_ok=True)
    srcs = _sources("host", ".cpp")
    hdrs = _headers("host")
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"],
           "-I" + os.path.join(CSRC, "host")]
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(BUILD, "host", os.path.basename(s) + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            jobs.append([CXX] + CXX_FLAGS + inc + ["-c", s, "-o", o])
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out.strip():
                print(out)
    if jobs or not os.path.exists(HOST_SO):
        _link([CXX, "-shared"], HOST_SO, objs + ["-pthread"])
    return HOST_SO


SANITIZERS = {"address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "thread": ["-fsanitize=thread"]}


def build_host_sanitized(kind: str, verbose=False) -> str:
    """The host library compiled with AddressSanitizer + UBSan (``address``) or ThreadSanitizer (``thread``) into
    ``build/host_<kind>/_gb200_host.so``.  Run the CPU tests against it with

        GB200_HOST_SO=<that file> LD_PRELOAD=$(g++ -print-file-name=lib{a,t}san.so) python -m pytest tests -m "not gpu"

    (the interpreter itself is not instrumented, so the sanitizer runtime has to be loaded first).  The compiler must
    ship the runtime it links against: set ``CXX=/usr/bin/g++`` when the default one is a wrapper without it."""
    import pybind11
    if kind not in SANITIZERS:
        raise ValueError("sanitizer must be one of " + ", ".join(SANITIZERS))
    out_dir = os.path.join(BUILD, "host_" + kind)
    os.makedirs(out_dir, exist_ok=True)
    flags = [f for f in CXX_FLAGS if f != "-O2"] + ["-O1", "-g", "-fno-omit-frame-pointer"] + SANITIZERS[kind]
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(CSRC, "host")]
    hdrs = _headers("host")
    jobs, objs = [], []
    for s in _sources("host", ".cpp"):
        o = os.path.join(out_dir, os.path.basename(s) + ".o")
        objs.append(o)
        if _newer([s] + hdrs, o):
            jobs.append([CXX] + flags + inc + ["-c", s, "-o", o])
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out.strip():
                print(out)
    target = os.path.join(out_dir, "_gb200_host.so")
    if jobs or not os.path.exists(target):
        _link([CXX, "-shared"] + SANITIZERS[kind], target, objs + ["-pthread"])
    return target


def build_cuda(verbose=False, force=False):
    os.makedirs(os.path.join(BUILD, "cuda"), exist_ok=True)
    srcs = _sources("cuda", ".cu")
    hdrs = _headers("cuda")
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(BUILD, "cuda", os.path.basename(s) + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            jobs.append(([NVCC] + NVCC_FLAGS + ["-I" + os.path.join(CSRC, "cuda"), "-c", s, "-o", o],
                         o + ".log"))
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        for out in ex.map(lambda j: _run(*j), jobs):
            if verbose and out.strip():
                print(out)
    if jobs or not os.path.exists(CUDA_SO):
        _link([NVCC, "-shared"], CUDA_SO, objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"])
    return CUDA_SO


def build_all(verbose=False, force=False):
    h = build_host(verbose, force)
    c = build_cuda(verbose, force)
    return h, c


def ptxas_report():
    """Collect the ``-Xptxas -v`` lines (registers / spills / smem) of the last CUDA build."""
    lines = []
    d = os.path.join(BUILD, "cuda")
    if os.path.isdir(d):
        for f in sorted(os.listdir(d)):
            if f.endswith(".log"):
                with open(os.path.join(d, f)) as fh:
                    lines.append("== " + f)
                    lines += [ln.rstrip() for ln in fh if "ptxas info" in ln or "Compiling entry" in ln]
    return "\n".join(lines)


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print(build_host_sanitized(sys.argv[sys.argv.index("--sanitize") + 1], verbose="-v" in sys.argv))
    else:
        force = "--force" in sys.argv
        print(build_all(verbose="-v" in sys.argv, force=force))
