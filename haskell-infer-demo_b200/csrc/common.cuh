/*
 * common.cuh - shared host/device helpers of libffn_int4.so: status reporting, BF16 helpers and
 * the one INT4 unpack routine every kernel (and the dequantize dump) goes through.
 */
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ffn_int4.h"

namespace ffn {

/* ---- status ------------------------------------------------------------------------------- */
int fail(int status, const char *fmt, ...);
void clear_error();
#define FFN_CUDA_TRY(expr, what)                                                              \
    do {                                                                                      \
        cudaError_t ffn_e_ = (expr);                                                          \
        if (ffn_e_ != cudaSuccess)                                                            \
            return ffn::fail(FFN_ERR_CUDA, "%s: %s", (what), cudaGetErrorString(ffn_e_));     \
    } while (0)

/* ---- BF16 --------------------------------------------------------------------------------- */
__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xFFFF0000u); }
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
/* round-to-nearest-even FP32 -> BF16 bits (same rule as csrc/linear_weight.cpp:34-44) */
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

/* ---- INT4 unpack -------------------------------------------------------------------------- */
/* The eight signed codes of one 32-bit word (nibble i = K index 8t+i, the layout of
 * csrc/kernels/gemm_quant.cu:45-48) as exact FP32 integers.  nibble^8 is code+8 in [0,15];
 * OR-ing it under the exponent of 2^23 gives 2^23 + code + 8 exactly, and the subtraction is
 * exact too, so float(code) here is bit-identical to an integer-to-float conversion. */
__device__ __forceinline__ void unpack8(uint32_t w, float c[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t n = ((w >> (4 * i)) & 0xFu) ^ 0x4B000008u;
        c[i] = __uint_as_float(n) - 8388616.0f;
    }
}

/* ---- loads -------------------------------------------------------------------------------- */
/* Streaming 16-byte weight load: read-only path, no L1 allocation (weights are read once). */
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

/* SiLU(g) * u with the reference's expression (csrc/kernels/silu.cu:70-72). */
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.0f + __expf(-g))) * u; }

}  // namespace ffn
