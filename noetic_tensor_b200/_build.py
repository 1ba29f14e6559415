"""Builds libnrl.so (the C-ABI CUDA library of include/nrl.h) in-tree with nvcc for sm_100a."""
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnrl.so")
SOURCES = ["nrl_api.cu", "nrl_bits.cu"]  # the second compiles the row kernels again for bit-packed masks
HEADERS = ["common.cuh", "row_fwd.cuh", "row_fwd_kernels.cuh", "row_fwd_group.cuh", "row_bwd.cuh", "token_ops.cuh", "ce_ops.cuh", "gumbel.cuh", "host_pack.cuh", "lane_ops.cuh", "readout.cuh", "row_api.inl"]
INCLUDE = os.path.join(os.path.dirname(HERE), "include", "nrl.h")


def source_hash():
    """First 16 hex digits of the SHA-256 of the kernel sources (part of nrl_key())."""
    h = hashlib.sha256()
    for f in SOURCES + HEADERS:
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    with open(INCLUDE, "rb") as fh:
        h.update(fh.read())
    return h.hexdigest()[:16]


def nvcc_path():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def up_to_date():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [INCLUDE, os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    common = [
        nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "--fmad=true", f'-DNRL_SRC_HASH="{source_hash()}"',
    ]
    if verbose:
        common.insert(1, "-Xptxas=-v")
    # one object per source, compiled side by side, then linked into the shared library
    objs, procs = [], []
    for src in SOURCES:
        obj = os.path.join(HERE, "build", os.path.splitext(src)[0] + ".o")
        os.makedirs(os.path.dirname(obj), exist_ok=True)
        objs.append(obj)
        procs.append(subprocess.Popen(common + ["-c", os.path.join(CSRC, src), "-o", obj], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    failed = False
    for pr in procs:
        out, err = pr.communicate()
        if pr.returncode != 0:
            sys.stderr.write(out + err)
            failed = True
        elif verbose:
            sys.stderr.write(err)
    if failed:
        raise RuntimeError("nvcc failed building libnrl.so")
    r = subprocess.run([nvcc_path(), "--shared", "-cudart", "static", "-o", LIB] + objs, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("nvcc failed linking libnrl.so")
    return LIB


HOST_HEADER = os.path.join(HERE, "host", "noetic_rl.hpp")


def build_host_program(source, out):
    """Compiles a C++ program that uses host/noetic_rl.hpp (the C++ mirror of `nn::rl`) and links
    it against libnrl.so and the CUDA runtime. g++ only: the header holds no device code."""
    build()
    deps = [source, HOST_HEADER, os.path.join(HERE, "host", "noetic_loss.hpp"), INCLUDE, LIB]
    if os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cuda = os.path.dirname(os.path.dirname(nvcc_path()))
    cmd = [
        "g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-I", os.path.join(cuda, "include"), source, "-o", out,
        "-L", HERE, "-l:libnrl.so", "-L", os.path.join(cuda, "lib64"), "-lcudart",
        "-Wl,-rpath,$ORIGIN/" + os.path.relpath(HERE, os.path.dirname(out)), "-Wl,-rpath," + os.path.join(cuda, "lib64"),
    ]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("g++ failed building " + os.path.basename(out))
    return out


if __name__ == "__main__":
    build(force=True, verbose="-v" in sys.argv)
    print(LIB)
