"""Builds libopenfish.so (C host layer + sm_100a kernels) and the `openfish` command-line driver
in-tree with nvcc and gcc.

    python -m openfish_b200.build            # build if sources are newer than the library
    python -m openfish_b200.build --force
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libopenfish.so")
CLI_SRC = os.path.join(HERE, "cli", "openfish_cli.c")
CLI = os.path.join(HERE, "bin", "openfish")  # the command-line driver, linked against LIB
CMP_SRC = os.path.join(HERE, "cli", "compare_blob.c")
CMP = os.path.join(HERE, "bin", "compare_blob")  # tensor-file comparison in the reference's format
CU = ["scan.cu", "beam_search.cu", "posterior_seq.cu", "rotary.cu", "decode_b200.cu", "decode_static.cu",
      "selfcheck.cu", "adaptor.cu"]
CC = ["openfish_api.c"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def _stale():
    if not os.path.exists(LIB) or not os.path.exists(CLI) or not os.path.exists(CMP):
        return True
    t = min(os.path.getmtime(LIB), os.path.getmtime(CLI), os.path.getmtime(CMP))
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [CLI_SRC, CMP_SRC]
    deps += [os.path.join(dp, f) for dp, _, fs in os.walk(os.path.join(ROOT, "include")) for f in fs]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    objs = []
    procs = []
    for f in CU:
        o = os.path.join(obj_dir, f + ".o")
        cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, f), "-o", o]
        procs.append((cmd, subprocess.Popen(cmd)))
        objs.append(o)
    for f in CC:
        o = os.path.join(obj_dir, f + ".o")
        cmd = ["gcc", "-O2", "-fPIC", "-Wall", "-std=gnu11", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
               "-c", os.path.join(CSRC, f), "-o", o]
        procs.append((cmd, subprocess.Popen(cmd)))
        objs.append(o)
    for cmd, p in procs:
        if p.wait() != 0:
            raise RuntimeError("build step failed: " + " ".join(cmd))
    link = [NVCC, "-shared", "-o", LIB] + objs + ["-cudart", "static", "-lm"]
    subprocess.run(link, check=True)
    os.makedirs(os.path.dirname(CLI), exist_ok=True)
    subprocess.run(["gcc", "-O2", "-Wall", "-std=gnu11", "-I", os.path.join(ROOT, "include"), CLI_SRC, "-o", CLI,
                    "-L", LIB_DIR, "-lopenfish", "-Wl,-rpath,$ORIGIN/../lib", "-lm"], check=True)
    subprocess.run(["gcc", "-O2", "-Wall", "-std=gnu11", CMP_SRC, "-o", CMP, "-lm"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
