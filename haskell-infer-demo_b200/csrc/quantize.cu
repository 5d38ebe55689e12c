/*
 * quantize.cu - the format's quantizer on the GPU: FP32 [N][K] in device memory -> packed nibbles
 * [N][K/2] and BF16 scales [N][K/128], byte-identical to the reference's CPU quantizer
 * (linear_quantize_int4, csrc/linear_weight.cpp:108-176), which its offline converter calls once per
 * tensor through a subprocess (scripts/quantize_weights.py:136-156).
 *
 * Arithmetic, in the reference's order and with IEEE operations (no fast-math, denormals kept):
 *   max_abs over the 128-group; scale = BF16_RNE(max_abs / 7), the all-zero group's scale = 1;
 *   q = clip(nearbyintf(w / scale), -7, 7) against the ROUNDED scale; low K index in the low nibble.
 * Refusals, also the reference's: a non-finite element; a group whose scale does not round to a
 * positive finite BF16 (e.g. a group of 1e-40).  The reference validates everything before it
 * writes anything; so does this file (one checking pass, then the writing pass).
 *
 * One warp per group: a lane loads four consecutive elements (one 16-byte load, 512 contiguous bytes
 * per warp), the maximum is a five-step shuffle, and each lane stores its two packed bytes.
 */
#include "common.cuh"
#include "kernels.h"

namespace ffn {

/* BF16 round-to-nearest-even by the reference's bit formula (csrc/linear_weight.cpp:34-45); the
 * inputs here are finite. */
__device__ __forceinline__ uint16_t bf16_rne_bits(float v) {
    uint32_t bits = __float_as_uint(v);
    bits += 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

struct QuantStatus {
    unsigned long long bad_element; /* 1 + index of a non-finite element, 0 = none */
    unsigned long long bad_group;   /* 1 + (row * groups + group) of an unrepresentable scale, 0 = none */
};

template <bool WRITE>
__global__ void __launch_bounds__(256) quantize_int4_kernel(const float *__restrict__ w, uint8_t *__restrict__ packed,
                                                            uint16_t *__restrict__ scales, long long groups_total,
                                                            QuantStatus *status) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long grp = warp; grp < groups_total; grp += nwarps) {
        const long long base = grp * FFN_INT4_GROUP + lane * 4;
        const float4 v = *(const float4 *)(w + base);
        const float e[4] = {v.x, v.y, v.z, v.w};
        float max_abs = 0.0f;
        bool finite = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            finite = finite && isfinite(e[i]);
            max_abs = fmaxf(max_abs, fabsf(e[i]));
        }
        if (!WRITE && !finite) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (!isfinite(e[i])) atomicMin(&status->bad_element, (unsigned long long)(base + i) + 1ull);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) max_abs = fmaxf(max_abs, __shfl_xor_sync(0xFFFFFFFFu, max_abs, o));
        const uint16_t scale_bits = max_abs == 0.0f ? (uint16_t)0x3F80u : bf16_rne_bits(__fdiv_rn(max_abs, 7.0f));
        const float scale = bf16_bits_to_f32(scale_bits);
        if (!WRITE) {
            if (lane == 0 && (!(scale > 0.0f) || !isfinite(scale))) atomicMin(&status->bad_group, (unsigned long long)grp + 1ull);
            continue;
        }
        if (lane == 0) scales[grp] = scale_bits;
        uint32_t nib[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float q = rintf(__fdiv_rn(e[i], scale)); /* nearest even, like nearbyintf in the default mode */
            q = fminf(fmaxf(q, -7.0f), 7.0f);
            nib[i] = (uint32_t)((int)q) & 0xFu;
        }
        const uint16_t two = (uint16_t)(nib[0] | (nib[1] << 4) | (nib[2] << 8) | (nib[3] << 12));
        *(uint16_t *)(packed + base / 2) = two;
    }
}

}  // namespace ffn

using namespace ffn;

extern "C" int ffn_quantize_int4(const void *weights, void *packed, void *scales, long long n, long long k, void *stream_) {
    clear_error();
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!weights || !packed || !scales) return fail(FFN_ERR_CONFIG, "ffn_quantize_int4: null argument");
    if (n <= 0 || k <= 0) return fail(FFN_ERR_CONFIG, "ffn_quantize_int4: [%lld, %lld] is not a weight shape", n, k);
    if (k % FFN_INT4_GROUP) return fail(FFN_ERR_CONFIG, "ffn_quantize_int4: K = %lld is not a whole number of %d-wide groups", k, FFN_INT4_GROUP);
    if (n % 8) return fail(FFN_ERR_CONFIG, "ffn_quantize_int4: N = %lld is not a multiple of the 8-row tile", n);
    if (((uintptr_t)weights & 15) || ((uintptr_t)packed & 1) || ((uintptr_t)scales & 1))
        return fail(FFN_ERR_CONFIG, "ffn_quantize_int4: weights must be 16-byte aligned, outputs 2-byte aligned");
    const long long groups = n * (k / FFN_INT4_GROUP);
    QuantStatus *status = nullptr;
    if (cudaMalloc(&status, sizeof(QuantStatus)) != cudaSuccess) { (void)cudaGetLastError(); return fail(FFN_ERR_ALLOC, "ffn_quantize_int4: cannot allocate the status words"); }
    int rc = FFN_OK;
    QuantStatus host;
    const unsigned grid = (unsigned)((groups + 7) / 8 < 148ll * 16 ? (groups + 7) / 8 : 148ll * 16);
    do {
        if (cudaMemsetAsync(status, 0xFF, sizeof(QuantStatus), stream) != cudaSuccess) { rc = fail(FFN_ERR_CUDA, "ffn_quantize_int4: memset failed"); break; }
        quantize_int4_kernel<false><<<grid, 256, 0, stream>>>((const float *)weights, nullptr, nullptr, groups, status);
        if (cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
            cudaStreamSynchronize(stream) != cudaSuccess) {
            rc = fail(FFN_ERR_CUDA, "ffn_quantize_int4: checking pass failed: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        if (host.bad_element != ~0ull) {
            rc = fail(FFN_ERR_WEIGHTS, "ffn_quantize_int4: element %llu is not finite; a quantizer cannot invent a scale for it",
                      host.bad_element - 1ull);
            break;
        }
        if (host.bad_group != ~0ull) {
            const unsigned long long g = host.bad_group - 1ull, per_row = (unsigned long long)(k / FFN_INT4_GROUP);
            rc = fail(FFN_ERR_WEIGHTS, "ffn_quantize_int4: row %llu group %llu rounds to a scale that is not positive and finite; "
                      "the format cannot represent it", g / per_row, g % per_row);
            break;
        }
        quantize_int4_kernel<true><<<grid, 256, 0, stream>>>((const float *)weights, (uint8_t *)packed, (uint16_t *)scales, groups, status);
        if (cudaGetLastError() != cudaSuccess || cudaStreamSynchronize(stream) != cudaSuccess)
            rc = fail(FFN_ERR_CUDA, "ffn_quantize_int4: writing pass failed");
    } while (0);
    cudaFree(status);
    return rc;
}
