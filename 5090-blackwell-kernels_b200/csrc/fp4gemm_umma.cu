// Tensor-core (tcgen05 block-scaled) route of the fp4 GEMM. Until the kernel lands this hook
// declines every shape and variant 2 runs the CUDA-core kernel.
#include "qgemm_simt.cuh"

namespace spk {
int fp4gemm_umma_try(const simt::Params&, int, cudaStream_t, bool* taken) {
    *taken = false;
    return SPK_OK;
}
}  // namespace spk
