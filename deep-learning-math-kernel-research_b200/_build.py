"""Compiles the library: csrc/*.cu for sm_100a into lib/libeuler_b200.so (nvcc cross-compiles without
a GPU; one object per translation unit, compiled in parallel, rebuilt when its source, a header or
the flags changed) and the C++ host library lib/libel.so, which exports the reference's own C++
symbols (eld_conv_t, elx_conv, reorder<>) on top of it.

This module does not load the library, so it can run while the library is missing or stale."""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
LIB_PATH = PKG_DIR / "lib" / "libeuler_b200.so"
HOST_LIB_PATH = PKG_DIR / "lib" / "libel.so"
CSRC = PKG_DIR / "csrc"
CU_SOURCES = ["elb_api.cu", "int8_conv.cu", "int8_conv2.cu", "wino.cu", "depthwise.cu", "misc.cu", "elb_multi.cu", "f32_small_ic.cu", "f32_rgb_umma.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"]


def reference_root() -> Path:
    """The reference project's tree (only its public headers are needed here): $EULER_REFERENCE, else a
    checkout named `reference` beside this repository.  $EULER_REFERENCE_INCLUDE may name the include
    directory itself."""
    if os.environ.get("EULER_REFERENCE_INCLUDE"):
        return Path(os.environ["EULER_REFERENCE_INCLUDE"]).parent
    return Path(os.environ.get("EULER_REFERENCE", ROOT.parent / "reference"))


def build(verbose: bool = False) -> Path:
    """See the module docstring.  Returns the path of the CUDA library."""
    LIB_PATH.parent.mkdir(exist_ok=True)
    headers = [p for p in CSRC.glob("*") if p.suffix in (".cuh", ".hpp", ".h")] + [ROOT / "include" / "euler_b200.h"]
    hdr_time = max(p.stat().st_mtime for p in headers)
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    extra = os.environ.get("ELB_NVCC_EXTRA", "").split()       # e.g. -DELB_TUNING for kernel experiments
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"] + extra
    # objects compiled with other flags (an experiment build) are never reused
    stamp = obj_dir / "flags.txt"
    same_flags = stamp.exists() and stamp.read_text() == " ".join(compile_flags)
    stamp.write_text(" ".join(compile_flags))
    jobs = []
    for name in CU_SOURCES:
        src, obj = CSRC / name, obj_dir / (Path(name).stem + ".o")
        if not same_flags or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            cmd = ["nvcc"] + compile_flags + ["-c", "-o", str(obj), str(src)]
            if verbose:
                print(" ".join(cmd))
            jobs.append(subprocess.Popen(cmd))
    for j in jobs:
        if j.wait() != 0:
            raise subprocess.CalledProcessError(j.returncode, j.args)
    objs = [obj_dir / (Path(n).stem + ".o") for n in CU_SOURCES]
    if jobs or not LIB_PATH.exists() or any(o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs):
        subprocess.check_call(["nvcc"] + NVCC_FLAGS + ["-o", str(LIB_PATH)] + [str(o) for o in objs])
    # The C++ host library defines the reference's own exported symbols and is therefore compiled
    # with the reference's public headers; where that tree is absent the prebuilt library is kept.
    host_src = PKG_DIR / "host" / "euler_host.cpp"
    ref_inc = reference_root() / "include"
    hdeps = [host_src, LIB_PATH, ROOT / "include" / "euler_b200.h"]
    if (ref_inc / "euler.hpp").exists() and (
            not HOST_LIB_PATH.exists() or any(p.stat().st_mtime > HOST_LIB_PATH.stat().st_mtime for p in hdeps)):
        cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-include", "string",
               "-include", "cstdint", f"-I{ref_inc}", f"-I{ROOT / 'include'}", "-o", str(HOST_LIB_PATH),
               str(host_src), f"-L{LIB_PATH.parent}", "-leuler_b200", "-Wl,-rpath,$ORIGIN"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return LIB_PATH


