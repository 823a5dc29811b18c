"""Build the CPU oracle and, when the reference checkout is present, the
reference's own quantize / MoE kernels for pinning.

TEST INFRASTRUCTURE ONLY: nothing in the shipped library depends on what this
script produces.

  oracle/_build/libcaif_oracle.so       gcc, from oracle/caif_oracle.c
  oracle/_ref/libcaif_ref_kernels.so    nvcc, from the reference's unmodified
                                        src/caif_cuda_kernels_quant.cu, _moe.cu,
                                        _attention_support.cu (router softmax) and
                                        _elementwise.cu, _optimizers.cu compiled where they lie,
                                        plus oracle/ref_shim.cu

Both outputs are binaries kept out of version control.  The second one is only
built where the reference sources exist; elsewhere a previously built copy is
used as is.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libcaif_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libcaif_ref_kernels.so")
# the reference checkout: CAIF_REFERENCE_ROOT, else a "reference" directory beside this repository
REFERENCE_ROOT = os.environ.get("CAIF_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "caif_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-fvisibility=hidden", "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_reference_kernels(force=False):
    """Returns the path of the library, or None when it cannot be had."""
    ref_src = os.path.join(REFERENCE_ROOT, "src")
    sources = [os.path.join(ref_src, "caif_cuda_kernels_quant.cu"),
               os.path.join(ref_src, "caif_cuda_kernels_moe.cu"),
               os.path.join(ref_src, "caif_cuda_kernels_attention_support.cu"),
               os.path.join(ref_src, "caif_cuda_kernels_elementwise.cu"),
               os.path.join(ref_src, "caif_cuda_kernels_optimizers.cu"),
               os.path.join(ref_src, "caif_cuda_kernels_activations.cu"),
               os.path.join(ref_src, "caif_cuda_kernels_normalization.cu")]
    shim = os.path.join(HERE, "ref_shim.cu")
    if not all(os.path.exists(s) for s in sources):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, sources + [shim]):
        return REF_SO
    if shutil.which("nvcc") is None:
        return REF_SO if os.path.exists(REF_SO) else None
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-DUSE_CAIF_CUDA=1",
           "-I", os.path.join(REFERENCE_ROOT, "include", "caif"),
           "-o", REF_SO, shim] + sources
    subprocess.check_call(cmd)
    return REF_SO


def main():
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference_kernels(force="--force" in sys.argv))


if __name__ == "__main__":
    main()
