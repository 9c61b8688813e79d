// Tensor-core (tcgen05) route of the fp8 GEMM. Until the kernel lands this hook declines every
// shape, and variant 3 runs the CUDA-core kernel.
#include "qgemm_simt.cuh"

namespace spk {
int fp8gemm_umma_try(const simt::Params&, bool, int, cudaStream_t, bool* taken) {
    *taken = false;
    return SPK_OK;
}
}  // namespace spk
