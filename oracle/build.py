#!/usr/bin/env python3
"""Build recipe for the checker code under oracle/.  TEST INFRASTRUCTURE ONLY.

  python oracle/build.py            # oracle/libfortis_oracle.so   (C port of the native forward, OpenMP)
                                    # oracle/_ref/libfortis_ref_zb.so and libfortis_ref_rt.so when the reference
                                    # checkout is present

oracle/_ref/ holds the REFERENCE's own generated gather/scatter kernels for the MOM6-ZB host
(mom6_zb/gather.cu, compiled where it lies, never copied) linked against oracle/ref_stubs.cu, which supplies the
three symbols that file expects from the rest of a fortisc build (mgpuStreamCreate, fortis_model_input,
fortis_model_output).  Flags follow the reference's own gather build: -fmad=false (driver/fortisc.sh:136).
The result only runs on a GPU box; GPU tests use it as a second, independent checker of gather/scatter.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: FORTIS_REFERENCE, else a directory named "reference" beside this repository
REF = os.environ.get("FORTIS_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _stale(out, srcs):
    return (not os.path.exists(out)) or any(os.path.getmtime(s) > os.path.getmtime(out) for s in srcs)


def build_port(verbose=True):
    src = os.path.join(HERE, "native_forward.c")
    out = os.path.join(HERE, "libfortis_oracle.so")
    if _stale(out, [src]):
        cmd = ["gcc", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", src, "-o", out, "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return out


def build_ref(verbose=True):
    """Returns the path of the built library, or None when the reference checkout is absent."""
    gsrc = os.path.join(REF, "mom6_zb", "gather.cu")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libfortis_ref_zb.so")
    if not os.path.exists(gsrc):
        return out if os.path.exists(out) else None
    stubs = os.path.join(HERE, "ref_stubs.cu")
    os.makedirs(out_dir, exist_ok=True)
    if _stale(out, [gsrc, stubs]):
        cmd = ["nvcc", "-O2", "-fmad=false", "-lineinfo"] + ARCH + ["-shared", "-Xcompiler", "-fPIC", gsrc, stubs,
               "-o", out, "-lcudart"]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return out


def build_ref_rt(verbose=True):
    """The reference's runtime compiled unchanged where it lies: runtime/fortis_rt.c (stream, pool, fortis_gemm ->
    cuBLAS SGEMM, fortis_conv3d -> cuDNN) + runtime/fortis_fft.cu (direct and FFT conv).  Used on the GPU box as the
    incumbent GPU path the benchmark is compared with, and as a second checker of fortis_gemm / fortis_conv3d.
    Returns the library path, or None when the reference checkout is absent."""
    rt = os.path.join(REF, "runtime", "fortis_rt.c")
    fft = os.path.join(REF, "runtime", "fortis_fft.cu")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libfortis_ref_rt.so")
    if not (os.path.exists(rt) and os.path.exists(fft)):
        return out if os.path.exists(out) else None
    os.makedirs(out_dir, exist_ok=True)
    if _stale(out, [rt, fft]):
        # fortis_rt.c is C (its entry names must stay unmangled: fortis_fft.cu and generated code call them), so it goes
        # through gcc; the .cu file through nvcc, which also links
        cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
        obj = os.path.join(out_dir, "fortis_rt.o")
        cmds = [["gcc", "-O2", "-fPIC", "-I" + cuda_inc, "-c", rt, "-o", obj],
                ["nvcc", "-O2", "-lineinfo"] + ARCH + ["-shared", "-Xcompiler", "-fPIC", fft, obj, "-o", out,
                 "-lcublas", "-lcudnn", "-lcufft", "-lcudart"]]
        for cmd in cmds:
            if verbose:
                print(" ".join(cmd))
            subprocess.run(cmd, check=True)
        os.remove(obj)
    return out


if __name__ == "__main__":
    print(build_port())
    print(build_ref())
    print(build_ref_rt())
