"""Build the reference's own layer classes for pinning and for the GPU comparator.

TEST INFRASTRUCTURE ONLY: nothing in the shipped library depends on what this script produces.

  oracle/_ref/libcaif_ref_layers.so   every translation unit of the reference (src/*.cpp with g++ -std=c++23,
                                      src/*.cu with nvcc for sm_100a, ise_lib/src/*.cpp), compiled unmodified
                                      where it lies in the reference checkout, plus oracle/ref_layers_shim.cpp,
                                      a C-linkage doorway onto CAIF_DeviceFrozenLinear, CAIF_DeviceLoRAAdapter
                                      and CAIF_DeviceMoEFrozenExpert.

The reference's own build system is not run.  Its one host BLAS call (cblas_sgemm,
src/caif_host_gemm.cpp) is satisfied by the OpenBLAS that ships inside SciPy, through a one-line header
written under oracle/_ref/include/ (the system has no OpenBLAS package); cuBLAS, cuBLAS-Lt and cuDNN come
from the CUDA toolkit and the image.  Objects are cached under oracle/_ref/obj/.  Only built where the
reference checkout exists; elsewhere a previously built library is used as is.
"""
import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
OBJ_DIR = os.path.join(REF_DIR, "obj")
INC_DIR = os.path.join(REF_DIR, "include")
LAYERS_SO = os.path.join(REF_DIR, "libcaif_ref_layers.so")
REFERENCE_ROOT = os.environ.get("CAIF_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
CUDA_INC = "/usr/local/cuda/include"

CBLAS_SHIM = """#pragma once
/* written by oracle/build_ref_layers.py: the one BLAS symbol the reference's host path uses, bound to SciPy's OpenBLAS */
#ifdef __cplusplus
extern "C" {
#endif
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void scipy_cblas_sgemm(enum CBLAS_ORDER, enum CBLAS_TRANSPOSE, enum CBLAS_TRANSPOSE, int, int, int, float,
                       const float *, int, const float *, int, float, float *, int);
#define cblas_sgemm scipy_cblas_sgemm
#ifdef __cplusplus
}
#endif
"""


def scipy_openblas():
    try:
        import scipy
    except Exception:
        return None
    libs = glob.glob(os.path.join(os.path.dirname(os.path.dirname(scipy.__file__)), "scipy.libs", "libscipy_openblas*.so"))
    return libs[0] if libs else None


def _compile(job):
    src, obj, cmd = job
    if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
        return None
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        return "%s\n%s" % (" ".join(cmd), res.stderr[-2000:])
    return None


def build(force=False, jobs=None):
    """Returns the path of the library, or None when it cannot be had."""
    src_dir = os.path.join(REFERENCE_ROOT, "src")
    if not os.path.isdir(src_dir):
        return LAYERS_SO if os.path.exists(LAYERS_SO) else None
    blas = scipy_openblas()
    if shutil.which("nvcc") is None or shutil.which("g++") is None or blas is None:
        return LAYERS_SO if os.path.exists(LAYERS_SO) else None
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(os.path.join(INC_DIR, "openblas"), exist_ok=True)
    with open(os.path.join(INC_DIR, "openblas", "cblas.h"), "w") as f:
        f.write(CBLAS_SHIM)
    includes = ["-I", os.path.join(REFERENCE_ROOT, "include"), "-I", os.path.join(REFERENCE_ROOT, "include", "caif"),
                "-I", os.path.join(REFERENCE_ROOT, "ise_lib", "include"),
                "-I", os.path.join(REFERENCE_ROOT, "ise_lib", "include", "ise_lib"), "-I", CUDA_INC, "-I", INC_DIR]
    cxx = ["g++", "-std=c++23", "-O1", "-fPIC", "-fopenmp", "-DUSE_CAIF_CUDA=1", "-w"] + includes
    nvcc = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-Xcompiler", "-fPIC",
            "-DUSE_CAIF_CUDA=1", "-w"] + includes
    shim = os.path.join(HERE, "ref_layers_shim.cpp")
    todo = []
    objs = []
    for src in sorted(glob.glob(os.path.join(src_dir, "*.cpp"))) + \
            sorted(glob.glob(os.path.join(REFERENCE_ROOT, "ise_lib", "src", "*.cpp"))) + [shim]:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-4] + ".o")
        objs.append(obj)
        todo.append((src, obj, cxx + ["-c", src, "-o", obj]))
    for src in sorted(glob.glob(os.path.join(src_dir, "*.cu"))):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".cu.o")
        objs.append(obj)
        todo.append((src, obj, nvcc + ["-c", src, "-o", obj]))
    if force:
        for _, obj, _ in todo:
            if os.path.exists(obj):
                os.remove(obj)
    with ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as pool:
        errors = [e for e in pool.map(_compile, todo) if e]
    if errors:
        raise RuntimeError("reference layers: %d translation units failed; first:\n%s" % (len(errors), errors[0]))
    newest = max(os.path.getmtime(o) for o in objs)
    if os.path.exists(LAYERS_SO) and os.path.getmtime(LAYERS_SO) >= newest:
        return LAYERS_SO
    blas_dir = os.path.dirname(blas)
    link = ["g++", "-shared", "-fopenmp", "-o", LAYERS_SO] + objs + [
        "-L/usr/local/cuda/lib64", "-lcublas", "-lcublasLt", "-lcudart", "-lcudnn", blas,
        "-Wl,-rpath," + blas_dir, "-Wl,-rpath,/usr/local/cuda/lib64", "-lpthread", "-ldl", "-lm"]
    subprocess.check_call(link)
    return LAYERS_SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
