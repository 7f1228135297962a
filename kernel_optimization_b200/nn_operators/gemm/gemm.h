// gemm<GemmKernel>: the reference's single __global__ entry for both GEMM families
// (nn_operators/gemm/gemm.h:11-21).  The kernel object decides the tiling; the launch supplies
// grid, GemmKernel::thread_per_block and GemmKernel::smem_total_size_in_bytes.
#pragma once

#include <type_traits>

#include "simt_gemm.h"
#include "tensor_core_compat.h"

template <typename GemmKernel>
__global__ void __launch_bounds__(GemmKernel::thread_per_block)
gemm(const shape::GemmCoord problem_size, typename GemmKernel::ElementA *ptr_A, typename GemmKernel::ElementB *ptr_B,
     typename GemmKernel::ElementC *ptr_C, typename GemmKernel::ElementC *ptr_D) {
    GemmKernel kernel;
    kernel(problem_size, ptr_A, ptr_B, ptr_C, ptr_D);
}
