"""Builds libdnxcu.so (CUDA kernels + C ABI + runtime) in-tree with nvcc for sm_100a.

Run as `python -m denox_b200.build`.  The shared library is written next to this
file; it is the only thing the Python layer loads.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libdnxcu.so")
SOURCES = ["api.cu", "kernels_mem.cu", "conv_direct.cu", "conv_tc.cu", "runtime.cu", "db.cu", "static_scratch.cu", "halo_xchg.cu", "select.cu", "supergraph.cu", "flatbuf.cu", "dnx.cu", "onnx.cu"]


def nvcc_path():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "dnxcu.h"),
                                                             os.path.join(HERE, "cli", "main.cpp")]
    if not os.path.exists(os.path.join(HERE, "dnxcu-cli")):
        return True
    return any(os.path.getmtime(d) > t for d in deps)


def source_digest():
    """SHA-256 over the kernel sources and the public header, in a fixed order: becomes part of every variant's
    identity (dnxcu_variant_sha256), so that a benchmark database never serves timings of other kernel code."""
    import hashlib
    h = hashlib.sha256()
    files = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".h")))
    for path in files + [os.path.join(ROOT, "include", "dnxcu.h")]:
        h.update(os.path.basename(path).encode() + b"\0")
        h.update(open(path, "rb").read())
    return h.hexdigest()


def build(force=False, verbose=False, debug_aids=False):
    if not force and not needs_build():
        return OUT
    objs = []
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    common = [
        nvcc_path(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        f'-DDNXCU_SOURCE_DIGEST="{source_digest()}"',
    ]
    if debug_aids:  # development only: time line tracing and load / MMA / store switches in the conv kernels
        common += ["-DDNXCU_DEBUG_AIDS"]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", os.path.join(CSRC, src), "-o", obj],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if out.strip():
            print(f"--- {src}\n{out}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc_path(), "-shared", "-o", OUT + ".tmp", "-gencode", "arch=compute_100a,code=sm_100a"] + objs + [
        "-cudart", "static"]
    subprocess.check_call(link)
    os.replace(OUT + ".tmp", OUT)
    build_cli()
    return OUT


CLI = os.path.join(HERE, "dnxcu-cli")


def build_cli():
    """The command line front door (cli/main.cpp): plain C++ over the C ABI, linked against the library next to it."""
    src = os.path.join(HERE, "cli", "main.cpp")
    cmd = [os.environ.get("CXX") or shutil.which("g++") or "g++", "-std=c++17", "-O2", "-Wall", "-I", os.path.join(ROOT, "include"),
           src, "-o", CLI + ".tmp", "-L", HERE, "-ldnxcu", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    os.replace(CLI + ".tmp", CLI)
    return CLI


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_aids="--debug-aids" in sys.argv))
