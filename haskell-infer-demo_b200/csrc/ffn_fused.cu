#include "common.cuh"
#include "kernels.h"

namespace ffn {

int gemm_int4_dispatch(const void *a, const void *packed, const void *scales, void *out, int M, int N,
                       int K, cudaStream_t stream) {
    return gemm_int4_generic(a, packed, scales, out, nullptr, M, N, K, stream);
}

int fused_ffn_try(cudaStream_t, const void *, void *, void *, const FfnMlpWeights *, int, int, int) {
    return FFN_NOT_ADMITTED;
}

}  // namespace ffn
