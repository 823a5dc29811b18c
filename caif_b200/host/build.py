"""Compile the C++23 host layer classes (caif_host.hpp, caif_safetensors.hpp + host_api.cpp) into
caif_b200/libcaif_host.so, linked against libcaifq.so and the CUDA runtime."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libcaif_host.so")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build(force=False):
    srcs = [os.path.join(HERE, "host_api.cpp")]
    deps = srcs + [os.path.join(HERE, "caif_host.hpp"), os.path.join(HERE, "caif_safetensors.hpp"),
                   os.path.join(ROOT, "include", "caifq.h")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(d) <= os.path.getmtime(LIB) for d in deps):
        return LIB
    cmd = ["g++", "-std=c++23", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-Wextra",
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"), "-o", LIB] + srcs + [
        "-L", PKG, "-l:libcaifq.so", "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
