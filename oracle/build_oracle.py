"""Build the test oracles. TEST INFRASTRUCTURE ONLY (never imported by the product path).

    python oracle/build_oracle.py [--ref-dir <reference checkout>]

1. oracle/liboracle.so     the CPU restatement oracle/fluke_oracle.c (gcc, OpenMP, AVX2/FMA,
                           -ffp-contract=off so only the explicit fmaf() calls fuse).
2. oracle/_ref/libfluke_ref_cpu.so   the reference's own src/nn_cpu.c + error.c + misc.c,
                           compiled where they lie under the reference checkout (gcc, -O2 as the
                           reference Makefile does). Pins the fp32 functions of the oracle.
3. oracle/_ref/libfluke_ref_cuda.so  the reference's own pure-CUDA kernels (src/nn_cuda.c with
                           src/nn_kernel_cuda.h, `nvcc -x cu`, sm_100a) + the CPU sources: the
                           on-GPU comparator for the memory-bound kernels.
Steps 2-3 run only when the reference checkout exists; their outputs stay in oracle/_ref/
(git-ignored). No reference source is copied.
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(HERE, "_ref")


def run(cmd):
    print(">>", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_port():
    out = os.path.join(HERE, "liboracle.so")
    src = os.path.join(HERE, "fluke_oracle.c")
    if os.path.isfile(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    # -mfma: the explicit fmaf() calls become the hardware instruction (same correctly rounded
    # result as the library routine, many times faster); -ffp-contract=off still keeps every
    # a*b+c that is NOT written as fmaf() unfused. -mf16c: hardware f16 <-> f32 conversion.
    run(["gcc", "-O3", "-mavx2", "-mfma", "-mf16c", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
         "-fno-math-errno", "-o", out, src, "-lm"])
    return out


def build_reference(ref_dir):
    src = os.path.join(ref_dir, "src")
    inc = os.path.join(ref_dir, "include")
    if not os.path.isfile(os.path.join(src, "nn_cpu.c")):
        print(f"reference checkout not found at {ref_dir}; skipping oracle/_ref")
        return
    os.makedirs(REF_OUT, exist_ok=True)
    cpu_srcs = [os.path.join(src, f) for f in ("nn_cpu.c", "error.c", "misc.c")]
    cpu_so = os.path.join(REF_OUT, "libfluke_ref_cpu.so")
    if not os.path.isfile(cpu_so):
        run(["gcc", "-g", "-Wall", "-O2", "-fPIC", "-shared", "-I", inc, "-o", cpu_so]
            + cpu_srcs + ["-lm", "-lpthread"])
    cuda_so = os.path.join(REF_OUT, "libfluke_ref_cuda.so")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(cuda_so) and os.path.isfile(nvcc):
        objs = []
        for f in cpu_srcs:
            o = os.path.join(REF_OUT, os.path.basename(f)[:-2] + ".o")
            run(["gcc", "-g", "-Wall", "-O2", "-fPIC", "-I", inc, "-DHAVE_CUDA=1",
                 "-I", "/usr/local/cuda/include", "-c", f, "-o", o])
            objs.append(o)
        cu_o = os.path.join(REF_OUT, "nn_cuda.o")
        arch = ["-gencode", "arch=compute_100a,code=sm_100a"]
        run([nvcc, "-x", "cu", "-g", "-O2", "-lineinfo"] + arch
            + ["-Xcompiler", "-fPIC", "-I", inc, "-DHAVE_CUDA=1", "-c",
               os.path.join(src, "nn_cuda.c"), "-o", cu_o])
        run([nvcc, "-shared"] + arch + ["-o", cuda_so] + objs + [cu_o,
            "-lm", "-lpthread", "-lcudart_static", "-lrt", "-ldl"])
        for o in objs + [cu_o]:
            os.remove(o)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-dir", default=os.environ.get("FLUKE_REFERENCE_DIR", ""),
                    help="checkout of the reference project (or set FLUKE_REFERENCE_DIR); without it only "
                         "oracle/liboracle.so is built")
    args = ap.parse_args()
    build_port()
    if args.ref_dir:
        build_reference(args.ref_dir)


if __name__ == "__main__":
    sys.exit(main())
