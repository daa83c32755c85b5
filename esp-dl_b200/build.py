"""Builds libespdl_b200.so (CUDA kernels + C ABI) and libespdl_b200_host.so (C++ host layer) in-tree with nvcc
for sm_100a.  nvcc cross-compiles without a GPU."""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build(verbose=False, force=False):
    csrc = os.path.join(HERE, "csrc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = glob.glob(os.path.join(csrc, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    jobs = []
    objs = []
    for src in sorted(glob.glob(os.path.join(csrc, "*.cu"))):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=8) as ex:
        for out in ex.map(_run, jobs):
            if verbose and out:
                print(out)
    lib = os.path.join(HERE, "libespdl_b200.so")
    if force or jobs or not os.path.exists(lib):
        _run([NVCC] + ARCH + ["-shared", "-o", lib] + objs + ["-ccbin", "/usr/bin/g++"])
    # host layer (C++17, links against the C ABI only)
    host = os.path.join(HERE, "host")
    host_srcs = sorted(glob.glob(os.path.join(host, "*.cpp")))
    host_lib = os.path.join(HERE, "libespdl_b200_host.so")
    if host_srcs and (force or _newer(host_lib, host_srcs + glob.glob(os.path.join(host, "*.hpp")) + headers + [lib])):
        _run(["/usr/bin/g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-o", host_lib] + host_srcs +
             ["-I" + os.path.join(HERE, "..", "include"), "-I" + host, "-L" + HERE, "-lespdl_b200", "-Wl,-rpath,$ORIGIN"])
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
