"""Builds libtdc_b200.so (the CUDA kernels and their C ABI) in-tree for sm_100a.

    python ppopp23-tdc_b200/build.py [--force] [--verbose]

Object files go to ppopp23-tdc_b200/build/, the library to
ppopp23-tdc_b200/tdc_b200/libtdc_b200.so.  A source is recompiled when it or a header is
newer than its object.  nvcc cross-compiles without a GPU.
"""
import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "tdc_b200", "libtdc_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-I", INCLUDE,
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libtdc_b200.so cannot be built")
    return exe


def _newest_header():
    times = [os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    times += [os.path.getmtime(os.path.join(INCLUDE, f)) for f in os.listdir(INCLUDE)]
    return max(times)


def _compile(src, obj, verbose):
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return r.stderr if verbose else ""


def build_debug_bounds():
    """libtdc_b200_bounds.so: the same library compiled with -DTDC_DEBUG_BOUNDS, in which every global access of the
    fp32 kernels checks its offset first and records a violation instead of making the access (tdc_debug_bounds_read).
    Load it with TDC_B200_LIB=<path>; slower, for tests and for hunting an index error without faulting a GPU."""
    out = os.path.join(HERE, "tdc_b200", "libtdc_b200_bounds.so")
    obj_dir = os.path.join(HERE, "build", "bounds")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr = _newest_header()
    jobs, objs = [], []
    for f in srcs:
        src, obj = os.path.join(CSRC, f), os.path.join(obj_dir, f[:-3] + ".o")
        objs.append(obj)
        if not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr):
            jobs.append((src, obj))

    def one(job):
        r = subprocess.run([_nvcc(), *NVCC_FLAGS, "-DTDC_DEBUG_BOUNDS", "-c", job[0], "-o", job[1]], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (job[0], r.stderr))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(one, jobs))
    if jobs or not os.path.exists(out):
        r = subprocess.run([_nvcc(), "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s" % r.stderr)
    return out


def build_profile(level=1):
    """libtdc_b200_profile.so: the library with the tensor-core kernels compiled as a measurement build
    (-DTDC_TC_PROFILE=level, see csrc/conv_tc_persist.cuh; exports tdc_tc_profile_read).  Level 1 marks the phases of a
    CTA and times the issuers without slowing the kernel; level 2 times every role.  `python kernel_bench.py phases`
    builds and loads it; the other objects are those of the normal build."""
    build()
    out = os.path.join(HERE, "tdc_b200", "libtdc_b200_profile.so")
    obj_dir = os.path.join(HERE, "build", "profile%d" % level)
    os.makedirs(obj_dir, exist_ok=True)
    src, obj = os.path.join(CSRC, "conv_tc.cu"), os.path.join(obj_dir, "conv_tc.o")
    if not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), _newest_header()):
        r = subprocess.run([_nvcc(), *NVCC_FLAGS, "-DTDC_TC_PROFILE=%d" % level, "-c", src, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (src, r.stderr))
    objs = [obj] + [os.path.join(OBJ, f[:-3] + ".o") for f in sorted(os.listdir(CSRC)) if f.endswith(".cu") and f != "conv_tc.cu"]
    r = subprocess.run([_nvcc(), "-shared", "-o", out, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s" % r.stderr)
    return out


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr = _newest_header()
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs, objs = [], []
    for f in srcs:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr):
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for out in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
                if out:
                    sys.stderr.write(out)
    if jobs or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    build_baseline_tool(force)
    build_layer_driver(force)
    build_rates_tool(force)
    return LIB


DRIVER_SRC = os.path.join(HERE, "drivers", "layer_driver.cu")
DRIVER_EXE = os.path.join(HERE, "tdc_b200", "layer_driver")


def build_layer_driver(force=False, defines=()):
    """The native per-shape layer driver (drivers/layer_driver.cu): a C++ program that calls the library through its C
    ABI only.  `defines` may carry the reference's compile-time macros, e.g. ("LAYER_C=64", "LAYER_N=64", "LAYER_H=56", "LAYER_W=56")."""
    newest = max(os.path.getmtime(DRIVER_SRC), os.path.getmtime(LIB), os.path.getmtime(os.path.join(INCLUDE, "tdc_b200.h")))
    if not force and not defines and os.path.exists(DRIVER_EXE) and os.path.getmtime(DRIVER_EXE) >= newest:
        return DRIVER_EXE
    cmd = [_nvcc(), "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", INCLUDE, DRIVER_SRC, "-o", DRIVER_EXE,
           "-L", os.path.dirname(LIB), "-ltdc_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"] + ["-D" + d for d in defines]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("layer_driver failed to build:\n%s\n%s" % (r.stdout, r.stderr))
    return DRIVER_EXE


RATES_SRC = os.path.join(HERE, "drivers", "tc_rates.cu")
RATES_EXE = os.path.join(HERE, "tdc_b200", "tc_rates")


def build_rates_tool(force=False):
    """drivers/tc_rates.cu: a standalone microbenchmark of the two per-SM rates that bound the tensor-core kernel (MMA
    issue from shared memory, bulk copies out of L2); links nothing of the library."""
    if not force and os.path.exists(RATES_EXE) and os.path.getmtime(RATES_EXE) >= os.path.getmtime(RATES_SRC):
        return RATES_EXE
    r = subprocess.run([_nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", RATES_SRC, "-o", RATES_EXE], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("tc_rates failed to build:\n%s\n%s" % (r.stdout, r.stderr))
    return RATES_EXE


BASELINE_SRC = os.path.join(HERE, "baselines", "cudnn_layer.cpp")
BASELINE_EXE = os.path.join(HERE, "tdc_b200", "cudnn_layer_baseline")


def build_baseline_tool(force=False):
    """The cuDNN algorithm baselines of the layer driver (a measurement tool, a process of its own; not part of the
    library).  Skipped with a note when the cuDNN headers are not installed."""
    inc = next((d for d in ("/usr/include/x86_64-linux-gnu", "/usr/include", "/usr/local/cuda/include")
                if os.path.exists(os.path.join(d, "cudnn.h"))), None)
    if inc is None:
        sys.stderr.write("cudnn.h not found: cudnn_layer_baseline not built\n")
        return None
    if not force and os.path.exists(BASELINE_EXE) and os.path.getmtime(BASELINE_EXE) >= os.path.getmtime(BASELINE_SRC):
        return BASELINE_EXE
    cmd = [_nvcc(), "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-I", inc, BASELINE_SRC, "-o", BASELINE_EXE,
           "-lcudnn", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write("cudnn_layer_baseline not built:\n%s\n" % r.stderr)
        return None
    return BASELINE_EXE


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--debug-bounds", action="store_true", help="also build the range-checked variant of the library")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    if a.debug_bounds:
        print(build_debug_bounds())
