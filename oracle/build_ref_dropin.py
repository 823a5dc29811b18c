"""Build the reference with its frozen-linear translation unit bound to libcaifq.so, and its own test programs.

TEST INFRASTRUCTURE ONLY.  Proof of the drop-in boundary: the reference's classes, callers and test
programs, compiled from its unmodified sources, run on this library's kernels.

  oracle/_ref/gen/caif_device_frozen_linear.cpp   generated, never committed: the reference's translation unit
                                                  with the definitions of ForwardImpl and BackwardImpl taken out
                                                  and oracle/ref_dropin/frozen_linear_bodies.inc (calls into the
                                                  C ABI) put in their place; everything else is the reference's text
  oracle/_ref/gen/caif_device_lora_adapter.cpp    generated likewise: the reference's two bodies renamed to
                                                  ...Reference (kept for base layers that are not frozen linears)
                                                  and oracle/ref_dropin/lora_adapter_bodies.inc appended
  oracle/_ref/gen/include/*.h                     copies of two reference headers with the added declarations
  oracle/_ref/libcaif_ref_dropin.so               all other reference objects (as built by build_ref_layers.py)
                                                  + the generated unit, linked against caif_b200/libcaifq.so
  oracle/_ref/bin/<test>                          the reference's own tests/test_device_frozen_linear.cpp,
                                                  test_device_lora_adapter.cpp, test_device_moe_frozen_expert.cpp,
                                                  test_pluggable_projections.cpp linked against that library
  oracle/_ref/bin/<test>_stock                    the same programs against the unmodified reference library

Run the programs on a box with a GPU with `python oracle/build_ref_dropin.py --run LOGDIR`.
Only built where the reference checkout exists; elsewhere the previously built files are used as they are.
"""
import os
import re
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)
import build_ref_layers as layers  # noqa: E402

REF_DIR = layers.REF_DIR
GEN_DIR = os.path.join(REF_DIR, "gen")
BIN_DIR = os.path.join(REF_DIR, "bin")
DROPIN_SO = os.path.join(REF_DIR, "libcaif_ref_dropin.so")
BODIES = os.path.join(HERE, "ref_dropin", "frozen_linear_bodies.inc")
LORA_BODIES = os.path.join(HERE, "ref_dropin", "lora_adapter_bodies.inc")
GEN_INC = os.path.join(GEN_DIR, "include")
TESTS = ("test_device_frozen_linear", "test_device_lora_adapter", "test_device_moe_frozen_expert",
         "test_pluggable_projections")
REPLACED = ("ForwardImpl", "BackwardImpl")


def _cut_function(text, name):
    """Remove the out-of-class definition of CAIF_DeviceFrozenLinear<...>::name: from the `template<` line
    before it to the closing brace in column 0 after it (the reference's layout)."""
    m = re.search(r"^template<typename ComputeT,typename StorageT>\n[^\n]*\n?CAIF_DeviceFrozenLinear<ComputeT,StorageT>::"
                  + name + r"\(", text, re.M)
    if m is None:
        raise RuntimeError("reference frozen linear: definition of %s not found" % name)
    end = text.index("\n}\n", m.end()) + 3
    return text[:m.start()] + text[end:]


def _gen_headers():
    """Copies of two reference headers with the declarations the bindings add: public, non-virtual members
    only, so the classes' layout and vtables are those every other translation unit sees."""
    os.makedirs(GEN_INC, exist_ok=True)
    inc = os.path.join(layers.REFERENCE_ROOT, "include", "caif")
    with open(os.path.join(inc, "caif_device_frozen_linear.h")) as f:
        text = f.read()
    anchor = "    bool IsPrefetched()const override{return _is_prefetched;}\n"
    at = text.index(anchor) + len(anchor)
    text = text[:at] + "    caifq_weight AsCaifq()const;   // codes, scales and dims as the C ABI takes them\n" + text[at:]
    text = text.replace('#include "caif_device_layer.h"\n', '#include "caifq.h"\n#include "caif_device_layer.h"\n', 1)
    with open(os.path.join(GEN_INC, "caif_device_frozen_linear.h"), "w") as f:
        f.write(text)
    with open(os.path.join(inc, "caif_device_lora_adapter.h")) as f:
        text = f.read()
    anchor = "    CAIF_DeviceTensor BackwardImpl(const CAIF_DeviceTensor &grad_output,CAIF_RunContext &ctx)override;\n"
    at = text.index(anchor) + len(anchor)
    text = (text[:at] +
            "    CAIF_DeviceTensor ForwardImplReference(const CAIF_DeviceTensor &input,CAIF_RunContext &ctx);\n"
            "    CAIF_DeviceTensor BackwardImplReference(const CAIF_DeviceTensor &grad_output,CAIF_RunContext &ctx);\n" +
            text[at:])
    with open(os.path.join(GEN_INC, "caif_device_lora_adapter.h"), "w") as f:
        f.write(text)


def generate():
    """Writes the generated translation units; returns their paths."""
    _gen_headers()
    src = os.path.join(layers.REFERENCE_ROOT, "src", "caif_device_frozen_linear.cpp")
    with open(src) as f:
        text = f.read()
    for name in REPLACED:
        text = _cut_function(text, name)
    with open(BODIES) as f:
        bodies = f.read()
    marker = "template class CAIF_DeviceFrozenLinear<float,float>;"
    at = text.index(marker)
    # the bodies go before the explicit instantiations, inside the reference's namespace
    text = text[:at] + bodies + "\n" + text[at:]
    os.makedirs(GEN_DIR, exist_ok=True)
    out = os.path.join(GEN_DIR, "caif_device_frozen_linear.cpp")
    with open(out, "w") as f:
        f.write(text)

    # the LoRA adapter: the reference's two bodies stay, under another name, as the path for other base layers
    src = os.path.join(layers.REFERENCE_ROOT, "src", "caif_device_lora_adapter.cpp")
    with open(src) as f:
        text = f.read()
    for name in REPLACED:
        old = "CAIF_DeviceLoRAAdapter<ComputeT,StorageT>::%s(" % name
        if text.count(old) != 1:
            raise RuntimeError("reference LoRA adapter: definition of %s not found" % name)
        text = text.replace(old, "CAIF_DeviceLoRAAdapter<ComputeT,StorageT>::%sReference(" % name)
    with open(LORA_BODIES) as f:
        bodies = f.read()
    marker = "template class CAIF_DeviceLoRAAdapter<float,float>;"
    at = text.index(marker)
    text = text[:at] + bodies + "\n" + text[at:]
    text = '#include "caifq.h"\n#include "caif_device_frozen_linear.h"\n' + text
    out_lora = os.path.join(GEN_DIR, "caif_device_lora_adapter.cpp")
    with open(out_lora, "w") as f:
        f.write(text)
    return [out, out_lora]


def _includes():
    r = layers.REFERENCE_ROOT
    return ["-I", os.path.join(r, "include"), "-I", os.path.join(r, "include", "caif"),
            "-I", os.path.join(r, "ise_lib", "include"), "-I", os.path.join(r, "ise_lib", "include", "ise_lib"),
            "-I", layers.CUDA_INC, "-I", layers.INC_DIR, "-I", os.path.join(ROOT, "include"),
            "-I", os.path.join(r, "tests")]


def build():
    """Returns the list of test programs, or [] when they cannot be had."""
    have = [os.path.join(BIN_DIR, t) for t in TESTS if os.path.exists(os.path.join(BIN_DIR, t))]
    if not os.path.isdir(os.path.join(layers.REFERENCE_ROOT, "src")):
        return have
    if layers.build() is None:
        return have
    libcaifq = os.path.join(ROOT, "caif_b200", "libcaifq.so")
    if not os.path.exists(libcaifq):
        raise RuntimeError("build caif_b200/libcaifq.so first (python -m caif_b200.build)")
    cxx = ["g++", "-std=c++23", "-O1", "-fPIC", "-fopenmp", "-DUSE_CAIF_CUDA=1", "-w"] + _includes()
    gen_objs = []
    for gen in generate():
        obj = gen[:-4] + ".o"
        # the generated header copies shadow the reference's for these two units only
        subprocess.check_call(cxx[:1] + ["-I", GEN_INC] + cxx[1:] + ["-c", gen, "-o", obj])
        gen_objs.append(obj)
    others = sorted(os.path.join(layers.OBJ_DIR, o) for o in os.listdir(layers.OBJ_DIR)
                    if o.endswith(".o") and o not in ("caif_device_frozen_linear.o", "caif_device_lora_adapter.o",
                                                      "ref_layers_shim.o"))
    blas = layers.scipy_openblas()
    rpaths = ["$ORIGIN", "$ORIGIN/../../caif_b200", os.path.dirname(blas), "/usr/local/cuda/lib64"]
    link = ["g++", "-shared", "-fopenmp", "-o", DROPIN_SO] + gen_objs + others + [
        "-L" + os.path.dirname(libcaifq), "-lcaifq", "-L/usr/local/cuda/lib64", "-lcublas", "-lcublasLt", "-lcudart",
        "-lcudnn", blas, "-lpthread", "-ldl", "-lm"] + ["-Wl,-rpath," + p for p in rpaths]
    subprocess.check_call(link)
    os.makedirs(BIN_DIR, exist_ok=True)

    def one(job):
        test, stock = job
        # (stock: the same program against the unmodified reference library, to tell a test that fails on this
        # box for its own reasons from one that fails because of the substitution)
        exe = os.path.join(BIN_DIR, test + ("_stock" if stock else ""))
        src = os.path.join(layers.REFERENCE_ROOT, "tests", test + ".cpp")
        harness = os.path.join(layers.REFERENCE_ROOT, "tests", "caif_test_harness.cpp")   # pass / fail bookkeeping
        cmd = cxx + [src, harness, "-o", exe, "-L" + REF_DIR, "-lcaif_ref_layers" if stock else "-lcaif_ref_dropin",
                     "-L" + os.path.dirname(libcaifq), "-lcaifq",
                     "-L/usr/local/cuda/lib64", "-lcudart", "-lcublas",
                     "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath,$ORIGIN/../../../caif_b200",
                     "-Wl,-rpath," + os.path.dirname(blas), "-Wl,-rpath,/usr/local/cuda/lib64"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("%s: %s" % (test, res.stderr[-3000:]))
        return exe

    with ThreadPoolExecutor(max_workers=8) as pool:
        return list(pool.map(one, [(t, False) for t in TESTS] + [(t, True) for t in TESTS]))


def run(log_dir):
    """Run the built programs (needs a GPU); one log per program, returns {name: exit code}."""
    os.makedirs(log_dir, exist_ok=True)
    codes = {}
    for test in list(TESTS) + [t + "_stock" for t in TESTS]:
        exe = os.path.join(BIN_DIR, test)
        if not os.path.exists(exe):
            codes[test] = None
            continue
        with open(os.path.join(log_dir, test + ".log"), "w") as f:
            codes[test] = subprocess.run([exe], stdout=f, stderr=subprocess.STDOUT, timeout=1200).returncode
    return codes


if __name__ == "__main__":
    if len(sys.argv) >= 3 and sys.argv[1] == "--run":
        print(run(sys.argv[2]))
    else:
        print(build())
