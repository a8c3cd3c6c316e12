// Registers the reference's decode GEMV host function (declared in the reference's kernel/cuda/gemv.h, compiled
// from the reference's own kernel/cuda/gemv_kernel.cu) as torch.ops.nq_reference.nanoquant_dyn_forward.
// A namespace of its own, so that this library can be loaded beside this repository's `binary_kernels` operators.
// Used only by `bench.py --mode refkernel` (the reference's CUDA kernels timed on the same GPU).
#include <torch/extension.h>

#include "cuda/gemv.h"   // found through -I <reference>/src/nanoquant/kernel

TORCH_LIBRARY(nq_reference, m) {
    m.def(
        "nanoquant_dyn_forward("
        "Tensor x, Tensor scale_g, Tensor Ubits, Tensor? scale_l, Tensor Vbits, Tensor scale_h, "
        "int num_thread_stage1=128, int num_thread_stage2=128, int num_row_per_warp_stage1=2, "
        "int num_row_per_warp_stage2=2, int num_acc_stage1=4, int num_acc_stage2=4, "
        "int num_pipeline_stage1=2, int num_pipeline_stage2=2) -> Tensor");
}

TORCH_LIBRARY_IMPL(nq_reference, CUDA, m) { m.impl("nanoquant_dyn_forward", &nanoquant_dyn_forward); }
