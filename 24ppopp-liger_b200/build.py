"""In-tree build of the CUDA library (sm_100a only) and of the host-side C++ runtime.

`build_all()` compiles every source under csrc/ into one shared library next to this file with
nvcc; nothing is installed outside the tree and no JIT cache is used, so the built file travels
with the source tree.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libliger_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared",
]


def _sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cc")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _deps():
    out = _sources()
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh"))]
    inc = os.path.join(os.path.dirname(HERE), "include")
    out += [os.path.join(inc, f) for f in os.listdir(inc)]
    return out


def needs_build():
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > t for p in _deps())


HOST = os.path.join(HERE, "host")
BIN_DIR = os.path.join(HERE, "bin")
MAIN_PATH = os.path.join(BIN_DIR, "liger_main")
MPIRUN_PATH = os.path.join(BIN_DIR, "liger_mpirun")
SHIM_PATH = os.path.join(HERE, "libliger_mpi_shim.so")


def build_host(force=False):
    """The serving executable (host/main.cu), the shared-memory MPI stand-in and its launcher."""
    os.makedirs(BIN_DIR, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    shim_src = os.path.join(HOST, "mpi_shim", "mpi_shim.cc")
    jobs = [
        (SHIM_PATH, [shim_src], ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", SHIM_PATH, shim_src, "-lrt", "-lpthread"]),
        (MPIRUN_PATH, [os.path.join(HOST, "mpi_shim", "liger_mpirun.cc")],
         ["g++", "-O2", "-std=c++17", "-o", MPIRUN_PATH, os.path.join(HOST, "mpi_shim", "liger_mpirun.cc")]),
        (MAIN_PATH, _deps() + [os.path.join(HOST, f) for f in os.listdir(HOST) if f.endswith((".h", ".cu"))] + [LIB_PATH],
         [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17",
          "-I", os.path.join(HOST, "mpi_shim"), "-o", MAIN_PATH, os.path.join(HOST, "main.cu"), shim_src,
          "-L", HERE, "-lliger_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/..", "-lrt", "-lpthread"]),
    ]
    for out, deps, cmd in jobs:
        if force or not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps if os.path.exists(d)):
            res = subprocess.run(cmd, cwd=HERE, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(" ".join(cmd) + " failed:\n" + res.stdout + res.stderr)
    return MAIN_PATH


def build_all(force=False, verbose=False):
    """Compile csrc/ -> libliger_b200.so. Returns the library path."""
    if not force and not needs_build():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built on this machine")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + _sources() + ["-lpthread"]
    res = subprocess.run(cmd, cwd=HERE, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build_all(force=True, verbose=True))
