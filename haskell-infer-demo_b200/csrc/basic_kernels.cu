/*
 * basic_kernels.cu - the shape-generic kernels of the INT4 FFN path: a streaming INT4 GEMM for
 * any token count, SiLU*up on the row-interleaved gate|up layout, Gemma RMSNorm, the residual
 * add and the dequantize dump.  The decode-shaped fused kernels live in ffn_fused.cu; these are
 * what the operator-level entry points fall back on for shapes the fused kernels do not admit
 * (they are still CUDA kernels - there is no CPU path).
 */
#include "common.cuh"
#include "kernels.h"

namespace ffn {

/* ------------------------------------------------------------------------------------------- */
/* Generic INT4 GEMM: out[m][n] = sum_k a[m][k] * code[n][k] * scale[n][k/128]                  */
/* (replaces gemv_int4_kernel and gemm_int4_tiled_kernel, csrc/kernels/gemm_quant.cu:65-200)    */
/* ------------------------------------------------------------------------------------------- */
constexpr int kRowsPerWarp = 4;
constexpr int kWarps = 8;
constexpr int kRowsPerBlock = kRowsPerWarp * kWarps;
constexpr int kChunkK = 4096; /* activation columns staged per pass */

template <int MT>
__global__ void __launch_bounds__(kWarps * 32)
gemm_int4_rows_kernel(const uint16_t *__restrict__ a, const uint8_t *__restrict__ packed,
                      const uint16_t *__restrict__ scales, uint16_t *__restrict__ out_bf16,
                      float *__restrict__ out_f32, int m0, int M, int N, int K) {
    extern __shared__ __align__(16) uint16_t xs[]; /* [MT][kc] bf16 */
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kRowsPerBlock + warp * kRowsPerWarp;
    const int groups = K / FFN_INT4_GROUP;
    const int mcount = min(MT, M - m0);

    float acc[kRowsPerWarp][MT];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += kChunkK) {
        const int kc = min(kChunkK, K - k0);
        __syncthreads();
        /* stage the activation slice: 8 bf16 (16 bytes) per thread per step */
        for (int i = threadIdx.x; i < MT * (kc / 8); i += blockDim.x) {
            const int m = i / (kc / 8), c = i % (kc / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < mcount) v = *(const uint4 *)(a + (size_t)(m0 + m) * K + k0 + c * 8);
            *(uint4 *)(xs + (size_t)m * kc + c * 8) = v;
        }
        __syncthreads();

        for (int c = lane; c < kc / 32; c += 32) { /* one 16-byte chunk = 32 codes */
            const int kbase = k0 + c * 32;
            uint4 w[kRowsPerWarp];
            float s[kRowsPerWarp];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
                const int row = min(row0 + r, N - 1);
                w[r] = ld_stream16(packed + (size_t)row * (K / 2) + kbase / 2);
                s[r] = bf16_bits_to_f32(scales[(size_t)row * groups + kbase / FFN_INT4_GROUP]);
            }
            float part[kRowsPerWarp][MT];
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) part[r][m] = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float xv[MT][8];
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint4 q = *(const uint4 *)(xs + (size_t)m * kc + c * 32 + j * 8);
                    xv[m][0] = bf16_lo(q.x); xv[m][1] = bf16_hi(q.x);
                    xv[m][2] = bf16_lo(q.y); xv[m][3] = bf16_hi(q.y);
                    xv[m][4] = bf16_lo(q.z); xv[m][5] = bf16_hi(q.z);
                    xv[m][6] = bf16_lo(q.w); xv[m][7] = bf16_hi(q.w);
                }
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r) {
                    const uint32_t word = j == 0 ? w[r].x : j == 1 ? w[r].y : j == 2 ? w[r].z : w[r].w;
                    float code[8];
                    unpack8(word, code);
#pragma unroll
                    for (int m = 0; m < MT; ++m)
#pragma unroll
                        for (int i = 0; i < 8; ++i) part[r][m] = fmaf(code[i], xv[m][i], part[r][m]);
                }
            }
            /* the 32 codes of a chunk share one group, so the scale is applied once per chunk */
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[r][m] = fmaf(part[r][m], s[r], acc[r][m]);
        }
    }

#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float v = warp_sum(acc[r][m]);
            const int row = row0 + r;
            if (lane == 0 && row < N && m < mcount) {
                if (out_bf16) out_bf16[(size_t)(m0 + m) * N + row] = f32_to_bf16_bits(v);
                if (out_f32) out_f32[(size_t)(m0 + m) * N + row] = v;
            }
        }
}

template <int MT>
static int launch_rows(const uint16_t *a, const uint8_t *packed, const uint16_t *scales,
                       uint16_t *out_bf16, float *out_f32, int m0, int M, int N, int K,
                       cudaStream_t stream) {
    const size_t smem = (size_t)MT * (size_t)min(kChunkK, K) * sizeof(uint16_t);
    if (smem > 48 * 1024) {
        FFN_CUDA_TRY(cudaFuncSetAttribute(gemm_int4_rows_kernel<MT>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                     "gemm_int4: shared-memory opt-in");
    }
    const unsigned grid = (unsigned)((N + kRowsPerBlock - 1) / kRowsPerBlock);
    gemm_int4_rows_kernel<MT><<<grid, kWarps * 32, smem, stream>>>(a, packed, scales, out_bf16,
                                                                   out_f32, m0, M, N, K);
    FFN_CUDA_TRY(cudaGetLastError(), "gemm_int4 launch");
    return FFN_OK;
}

int gemm_int4_generic(const void *a, const void *packed, const void *scales, void *out_bf16,
                      float *out_f32, int M, int N, int K, cudaStream_t stream) {
    const uint16_t *ap = (const uint16_t *)a;
    const uint8_t *pp = (const uint8_t *)packed;
    const uint16_t *sp = (const uint16_t *)scales;
    uint16_t *ob = (uint16_t *)out_bf16;
    int m0 = 0;
    while (m0 < M) {
        const int left = M - m0;
        int st;
        if (left >= 8) { st = launch_rows<8>(ap, pp, sp, ob, out_f32, m0, M, N, K, stream); m0 += 8; }
        else if (left >= 4) { st = launch_rows<4>(ap, pp, sp, ob, out_f32, m0, M, N, K, stream); m0 += 4; }
        else if (left >= 2) { st = launch_rows<2>(ap, pp, sp, ob, out_f32, m0, M, N, K, stream); m0 += 2; }
        else { st = launch_rows<1>(ap, pp, sp, ob, out_f32, m0, M, N, K, stream); m0 += 1; }
        if (st != FFN_OK) return st;
    }
    return FFN_OK;
}

/* ------------------------------------------------------------------------------------------- */
/* SiLU * up on the row-interleaved layout (replaces silu_mul_packed_kernel, silu.cu:61-74)     */
/* ------------------------------------------------------------------------------------------- */
__global__ void silu_mul_packed_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ packed,
                                       int tokens, int inter) {
    const int t = blockIdx.y;
    if (t >= tokens) return;
    const uint16_t *row = packed + (size_t)t * 2 * inter;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inter; i += gridDim.x * blockDim.x) {
        const float g = bf16_bits_to_f32(row[i]);
        const float u = bf16_bits_to_f32(row[inter + i]);
        out[(size_t)t * inter + i] = f32_to_bf16_bits(silu_mul(g, u));
    }
}

int silu_mul_packed(void *out, const void *packed, int tokens, int inter, cudaStream_t stream) {
    const dim3 grid((unsigned)((inter + 255) / 256), (unsigned)tokens);
    silu_mul_packed_kernel<<<grid, 256, 0, stream>>>((uint16_t *)out, (const uint16_t *)packed,
                                                     tokens, inter);
    FFN_CUDA_TRY(cudaGetLastError(), "silu_mul_packed launch");
    return FFN_OK;
}

/* ------------------------------------------------------------------------------------------- */
/* Gemma RMSNorm (replaces the FlashInfer call in csrc/kernels/flashinfer_norm.cu:22-44).        */
/* Definition pinned by tests/test_library_ops.py:55-57: bf16(x * rsqrt(mean(x^2)+eps) * (1+w)). */
/* ------------------------------------------------------------------------------------------- */
__global__ void __launch_bounds__(256)
gemma_rms_norm_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ x,
                      const uint16_t *__restrict__ w, int cols, float eps, int gemma) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * cols;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = bf16_bits_to_f32(x[base + i]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += red[i];
    const float inv = rsqrtf(total / (float)cols + eps);
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = bf16_bits_to_f32(x[base + i]);
        const float g = bf16_bits_to_f32(w[i]) + (gemma ? 1.0f : 0.0f);
        out[base + i] = f32_to_bf16_bits(v * inv * g);
    }
}

/* ------------------------------------------------------------------------------------------- */
/* Residual update + norm in one pass (replaces kernel_residual_norm,                            */
/* csrc/kernels/flashinfer_norm.cu:112-174): r = bf16(r + sublayer) is stored, and the norm reads */
/* the ROUNDED r, as the next sublayer will.  The row stays in registers between the passes.      */
/* ------------------------------------------------------------------------------------------- */
constexpr int kResNormPerThread = 32; /* 256 threads x 32 elements: rows of up to 8192 stay in registers */
__global__ void __launch_bounds__(256)
residual_norm_kernel(uint16_t *__restrict__ normed, uint16_t *__restrict__ residual,
                     const uint16_t *__restrict__ sublayer, const uint16_t *__restrict__ w, int cols, float eps, int gemma) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * cols;
    const bool in_regs = cols <= 256 * kResNormPerThread;
    float keep[kResNormPerThread];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kResNormPerThread; ++j) {
        const int i = threadIdx.x + j * 256;
        keep[j] = 0.0f;
        if (in_regs && i < cols) {
            const uint16_t r = f32_to_bf16_bits(bf16_bits_to_f32(residual[base + i]) + bf16_bits_to_f32(sublayer[base + i]));
            residual[base + i] = r;
            keep[j] = bf16_bits_to_f32(r);
            ss = fmaf(keep[j], keep[j], ss);
        }
    }
    if (!in_regs)
        for (int i = threadIdx.x; i < cols; i += 256) {
            const uint16_t r = f32_to_bf16_bits(bf16_bits_to_f32(residual[base + i]) + bf16_bits_to_f32(sublayer[base + i]));
            residual[base + i] = r;
            const float v = bf16_bits_to_f32(r);
            ss = fmaf(v, v, ss);
        }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += red[i];
    const float inv = rsqrtf(total / (float)cols + eps);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < kResNormPerThread; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < cols) normed[base + i] = f32_to_bf16_bits(keep[j] * inv * (bf16_bits_to_f32(w[i]) + (gemma ? 1.0f : 0.0f)));
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += 256) /* this thread re-reads only what it stored itself */
            normed[base + i] = f32_to_bf16_bits(bf16_bits_to_f32(residual[base + i]) * inv * (bf16_bits_to_f32(w[i]) + (gemma ? 1.0f : 0.0f)));
    }
}

int residual_norm(void *normed, void *residual, const void *sublayer, const void *w, int cols, int rows, float eps,
                  int gemma, cudaStream_t stream) {
    residual_norm_kernel<<<rows, 256, 0, stream>>>((uint16_t *)normed, (uint16_t *)residual, (const uint16_t *)sublayer,
                                                   (const uint16_t *)w, cols, eps, gemma);
    FFN_CUDA_TRY(cudaGetLastError(), "residual_norm launch");
    return FFN_OK;
}

/* ------------------------------------------------------------------------------------------- */
/* SiLU(gate) * up over a contiguous [gate[n] | up[n]] buffer (replaces kernel_silu_mul,         */
/* csrc/kernels/silu.cu:29-52, which forwards to FlashInfer's act_and_mul): FP32, one rounding.  */
/* ------------------------------------------------------------------------------------------- */
__global__ void silu_mul_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ gate, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] = f32_to_bf16_bits(silu_mul(bf16_bits_to_f32(gate[i]), bf16_bits_to_f32(gate[n + i])));
}

int silu_mul_pair(void *out, const void *gate, int n, cudaStream_t stream) {
    silu_mul_kernel<<<(unsigned)min((n + 255) / 256, 1184), 256, 0, stream>>>((uint16_t *)out, (const uint16_t *)gate, n);
    FFN_CUDA_TRY(cudaGetLastError(), "silu_mul launch");
    return FFN_OK;
}

int gemma_rms_norm(void *out, const void *x, const void *w, int cols, int rows, float eps, int gemma,
                   cudaStream_t stream) {
    gemma_rms_norm_kernel<<<rows, 256, 0, stream>>>((uint16_t *)out, (const uint16_t *)x,
                                                    (const uint16_t *)w, cols, eps, gemma);
    FFN_CUDA_TRY(cudaGetLastError(), "gemma_rms_norm launch");
    return FFN_OK;
}

/* ------------------------------------------------------------------------------------------- */
/* Residual add (replaces residual_add_kernel, csrc/kernels/gdn_norm.cu:121-129)                 */
/* ------------------------------------------------------------------------------------------- */
__global__ void residual_add_kernel(uint16_t *__restrict__ dst, const uint16_t *__restrict__ src, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    dst[i] = f32_to_bf16_bits(bf16_bits_to_f32(dst[i]) + bf16_bits_to_f32(src[i]));
}

int residual_add(void *dst, const void *src, int n, cudaStream_t stream) {
    residual_add_kernel<<<(n + 255) / 256, 256, 0, stream>>>((uint16_t *)dst, (const uint16_t *)src, n);
    FFN_CUDA_TRY(cudaGetLastError(), "residual_add launch");
    return FFN_OK;
}

/* ------------------------------------------------------------------------------------------- */
/* Dequantize dump: float(code) * float(scale) through the kernels' own unpack routine          */
/* ------------------------------------------------------------------------------------------- */
__global__ void dequantize_kernel(float *__restrict__ out, const uint8_t *__restrict__ packed,
                                  const uint16_t *__restrict__ scales, long long words, int K,
                                  int *__restrict__ bad) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; /* one 32-bit word */
    if (i >= words) return;
    const uint32_t w = ((const uint32_t *)packed)[i];
    const long long e0 = i * 8;
    const long long row = e0 / K;
    const int k = (int)(e0 % K);
    const float s = bf16_bits_to_f32(scales[row * (K / FFN_INT4_GROUP) + k / FFN_INT4_GROUP]);
    float c[8];
    unpack8(w, c);
    int reserved = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        reserved += ((w >> (4 * j)) & 0xFu) == 0x8u;
        out[e0 + j] = c[j] * s;
    }
    if (reserved && bad) atomicAdd(bad, reserved);
}

int dequantize_int4(void *out, const void *packed, const void *scales, int N, int K, int *bad,
                    cudaStream_t stream) {
    const long long words = (long long)N * K / 8;
    if (bad) FFN_CUDA_TRY(cudaMemsetAsync(bad, 0, sizeof(int), stream), "dequantize: clear counter");
    dequantize_kernel<<<(unsigned)((words + 255) / 256), 256, 0, stream>>>(
        (float *)out, (const uint8_t *)packed, (const uint16_t *)scales, words, K, bad);
    FFN_CUDA_TRY(cudaGetLastError(), "dequantize launch");
    return FFN_OK;
}

}  // namespace ffn
