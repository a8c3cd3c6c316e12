"""Compile the reference's decode GEMV (its own ``kernel/cuda/gemv_kernel.cu``, from where it lies) into
``baseline/_ref/libnq_reference_kernels.so`` for sm_100, with the flags of the reference's ``kernel/setup.py:37-52``.

The reference's build is a torch CUDAExtension for the local GPU; this recipe runs the same compiler on the same file
with the same flags and links it with a small registration file of this repository (``ref_gemv_binding.cpp``), so the
library can travel to a GPU box.  Nothing of the reference is copied into the repository; the output directory is
git-ignored.  Usage: ``python baseline/build_ref_kernels.py [path of the reference checkout]``.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libnq_reference_kernels.so")


def build(reference_root: str) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    kdir = os.path.join(reference_root, "src", "nanoquant", "kernel")
    src = os.path.join(kdir, "cuda", "gemv_kernel.cu")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{kdir}",
                                                    "-I/usr/local/cuda/include"]
    abi = [f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    obj_k = os.path.join(OUT_DIR, "gemv_kernel.o")
    obj_b = os.path.join(OUT_DIR, "ref_gemv_binding.o")
    subprocess.run([nvcc, "-O3", "--use_fast_math", "-std=c++17", "-t", "32", "-gencode=arch=compute_100,code=sm_100",
                    "-Xcompiler", "-fPIC", *inc, *abi, "-c", src, "-o", obj_k], check=True)
    subprocess.run(["g++", "-O3", "-std=c++17", "-fPIC", *inc, *abi, "-c", os.path.join(HERE, "ref_gemv_binding.cpp"),
                    "-o", obj_b], check=True)
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    subprocess.run(["g++", "-shared", "-o", LIB, obj_k, obj_b, f"-L{tlib}", "-L/usr/local/cuda/lib64", "-lc10", "-lc10_cuda",
                    "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"], check=True)
    for obj in (obj_k, obj_b):   # only the library travels
        os.remove(obj)
    return LIB


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NANOQUANT_REFERENCE", os.path.join(os.sep, "root", "reference"))))
