/*
 * ffn_mma.cu - the batched INT4 FFN (3 <= M <= 64 tokens per pass) on the tensor cores.
 *
 * The reference keeps every M > 1 on cuBLAS BF16 because its SIMT tiled INT4 kernel measured 8-30x
 * slower (csrc/kernels/layers.cu:120-126; gemm_int4_tiled_kernel, csrc/kernels/gemm_quant.cu:65-157).
 * Here the packed weights stay the only weight traffic at M > 1 as well:
 *
 *   swap-AB: the WEIGHT rows fill the MMA's 16-wide M dimension, the tokens its 8-wide N dimension,
 *   so a batch of 8 tokens wastes nothing (mma.sync.m16n8k16, BF16 x BF16 -> FP32).
 *   One logic op turns two nibbles into two BF16 values 136+code ((w>>4s & 0x000F000F) ^ 0x43084308),
 *   one packed BF16 subtract makes them the exact integer codes; codes times BF16 activations are
 *   exact products, accumulated in FP32 inside the tensor core over one 128-wide group, and the group's
 *   FP32 scale is applied to that partial sum - the arithmetic of the reference's tiled kernel
 *   (gemm_quant.cu:134-147: slice = sum code*x, acc += slice*scale), so dequantisation stays exact.
 *
 * K order inside an MMA is free as long as A and B agree.  Lane (g, t) of a warp takes word 4j+t of a
 * row's 16-word group for the two MMAs of "virtual block" j; its B registers are then the eight
 * activations k = 8(4j+t) .. +7 in the order (0,4),(1,5),(2,6),(3,7), which is how the activations are
 * laid out in memory for this path (permute8: within every run of 8, element e sits at 2(e&3)+(e>>2)),
 * so one 16-byte shared load feeds both MMAs.
 *
 * Two launches per FFN: gate/up + SiLU*up (writes act, natural order for the caller and permuted for
 * the next launch), then down with the cross-rank exchange in its epilogue (same slot / flag protocol
 * as the fused decode kernel: CTA c of every rank owns the same 32 output rows).
 */
#include "common.cuh"
#include "kernels.h"

namespace ffn {

constexpr int kMmaWarps = 4;          /* one 128-wide group of the K chunk each */
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaRows = 32;          /* weight rows per CTA: two 16-row MMA tiles */
constexpr int kMmaKC = 512;           /* K per pipeline stage: 4 groups */
constexpr int kWRowBytes = kMmaKC / 2 + 16;   /* 272: conflict-free 32-bit reads down 8 rows */

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
/* nibbles s and s+4 of a word as exact BF16 codes (low half: nibble s, high half: nibble s+4) */
__device__ __forceinline__ uint32_t codes_bf16x2(uint32_t w, int s) {
    uint32_t v, d;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43084308, 0x6A;" : "=r"(v) : "r"(w >> (4 * s)));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(v), "r"(0x43084308u)); /* (136 + c) - 136 */
    return d;
}
__host__ __device__ __forceinline__ int permute8(int k) { /* position of element k in the permuted layout */
    const int e = k & 7;
    return (k & ~7) | (((e & 3) << 1) | (e >> 2));
}

struct MmaParams {
    const uint16_t *x;        /* activations, permuted layout, bf16 [M][K] */
    const uint8_t *w;         /* packed rows [N][K/2] */
    const uint16_t *s;        /* scales [N][K/128] */
    int M, N, K;              /* tokens (<= 8*NT), weight rows of this launch's matrix, columns */
    int up_offset;            /* gate/up: row index of up row 0; 0 for down */
    uint16_t *act;            /* gate/up: bf16 [M][N] natural order */
    uint16_t *act_perm;       /* gate/up: bf16 [M][N] permuted order (input of the down launch) */
    uint16_t *out;            /* down: bf16 [M][N] */
    uint16_t *residual;       /* down: optional bf16 [M][N], h <- bf16(h + y) */
    /* tensor parallelism (down only) */
    int tp, rank, slot_stride;
    unsigned long long *const *peer_slots;
    unsigned *tp_seq;
    unsigned *status;         /* word 3 of the device's synchronisation words */
};

/* One CTA: 32 weight rows (two tiles: [gate16 | up16] or down32) x all tokens, K streamed in 512-wide
 * chunks through a cp.async ring; warp ks takes group ks of every chunk for both tiles.  On return
 * red[(ks*32 + row) * ldr + token] holds the warps' FP32 partial sums. */
template <int NT, bool PAIRS>
__device__ __forceinline__ void mma_block(const MmaParams &P, int row0, uint8_t *smem, int stages, float *red, int ldr) {
    const int tid = threadIdx.x, lane = tid & 31, ks = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int xrow = kMmaKC * 2 + 64;                     /* bytes per token row of a stage, = 64 mod 128 */
    const int stage_bytes = kMmaRows * kWRowBytes + NT * 8 * xrow;
    const int G = P.K / FFN_INT4_GROUP;
    const int nchunks = (P.K + kMmaKC - 1) / kMmaKC;
    const uint32_t sbase = smem_addr(smem);

    auto row_of = [&](int r) -> int { /* global weight row of local row r */
        return PAIRS ? (r < 16 ? row0 + r : P.up_offset + row0 + (r - 16)) : row0 + r;
    };
    /* Each thread copies the same pieces of every chunk: 4 weight pieces (row r = i/16, 16-byte column
     * c = i%16) and NT*4 activation pieces (token m = i/64, column c = i%64).  Sources and shared
     * offsets are fixed per thread, so a chunk costs one add per piece. */
    const uint8_t *wsrc[4];
    uint32_t wdst[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int i = tid + q * kMmaThreads, r = i >> 4, c = i & 15;
        wsrc[q] = P.w + (size_t)row_of(r) * (P.K / 2) + c * 16;
        wdst[q] = (uint32_t)(r * kWRowBytes + c * 16);
    }
    const uint16_t *xsrc[NT * 4];
    uint32_t xdst[NT * 4];
#pragma unroll
    for (int q = 0; q < NT * 4; ++q) {
        const int i = tid + q * kMmaThreads, m = i >> 6, c = i & 63;
        xsrc[q] = m < P.M ? P.x + (size_t)m * P.K + c * 8 : nullptr;
        xdst[q] = (uint32_t)(kMmaRows * kWRowBytes + m * xrow + c * 16);
    }
    const int tcol_w = (tid & 15) * 32, tcol_x = (tid & 63) * 8; /* first K index of this thread's pieces */
    auto issue = [&](int chunk) {
        const uint32_t st = sbase + (uint32_t)(chunk % stages) * stage_bytes;
        const int k0 = chunk * kMmaKC, kc = min(kMmaKC, P.K - k0);
        if (tcol_w < kc) {
#pragma unroll
            for (int q = 0; q < 4; ++q) cp_async16(st + wdst[q], wsrc[q] + k0 / 2);
        }
        if (tcol_x < kc) {
#pragma unroll
            for (int q = 0; q < NT * 4; ++q)
                if (xsrc[q]) cp_async16(st + xdst[q], xsrc[q] + k0);
        }
        cp_async_commit();
    };

    /* tokens beyond M: zero their shared rows once (cp.async never writes them) */
    for (int s = 0; s < stages; ++s)
        for (int i = tid; i < (NT * 8 - P.M) * (xrow / 16); i += kMmaThreads) {
            const int m = P.M + i / (xrow / 16), c = i % (xrow / 16);
            *(uint4 *)(smem + (size_t)s * stage_bytes + kMmaRows * kWRowBytes + m * xrow + c * 16) = make_uint4(0, 0, 0, 0);
        }

    float acc[2][NT][4];
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[rt][n][i] = 0.0f;

    for (int c = 0; c < stages - 1; ++c) {
        if (c < nchunks) issue(c); else cp_async_commit();
    }
    for (int c = 0; c < nchunks; ++c) {
        /* chunk c was committed `stages - 1` groups ago: all but the newest stages-2 groups must be done */
        if (stages == 4) cp_async_wait<2>(); else if (stages == 3) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads(); /* everyone sees chunk c, and everyone is done with the buffer refilled below */
        if (c + stages - 1 < nchunks) issue(c + stages - 1); else cp_async_commit();
        const int grp = c * (kMmaKC / FFN_INT4_GROUP) + ks; /* this warp's group of the chunk */
        if (grp < G) {
            const uint32_t st = sbase + (uint32_t)(c % stages) * stage_bytes;
            const uint32_t xs = st + kMmaRows * kWRowBytes + (uint32_t)g * xrow + (uint32_t)ks * 256;
            float sc[2][2];
#pragma unroll
            for (int rt = 0; rt < 2; ++rt) {
                sc[rt][0] = bf16_bits_to_f32(__ldg(P.s + (size_t)row_of(rt * 16 + g) * G + grp));
                sc[rt][1] = bf16_bits_to_f32(__ldg(P.s + (size_t)row_of(rt * 16 + g + 8) * G + grp));
            }
            float part[2][NT][4];
#pragma unroll
            for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) part[rt][n][i] = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a[2][2][4]; /* [tile][mma of the pair][a0..a3] */
#pragma unroll
                for (int rt = 0; rt < 2; ++rt) {
                    const uint32_t wa = st + (uint32_t)(rt * 16 + g) * kWRowBytes + (uint32_t)ks * 64 + (uint32_t)(4 * j + t) * 4;
                    const uint32_t w_lo = lds32(wa), w_hi = lds32(wa + 8 * kWRowBytes); /* rows g and g+8 */
                    a[rt][0][0] = codes_bf16x2(w_lo, 0); a[rt][0][1] = codes_bf16x2(w_hi, 0);
                    a[rt][0][2] = codes_bf16x2(w_lo, 1); a[rt][0][3] = codes_bf16x2(w_hi, 1);
                    a[rt][1][0] = codes_bf16x2(w_lo, 2); a[rt][1][1] = codes_bf16x2(w_hi, 2);
                    a[rt][1][2] = codes_bf16x2(w_lo, 3); a[rt][1][3] = codes_bf16x2(w_hi, 3);
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint4 b = lds128(xs + (uint32_t)n * 8 * xrow + (uint32_t)(4 * j + t) * 16);
#pragma unroll
                    for (int rt = 0; rt < 2; ++rt) {
                        mma_bf16(part[rt][n], a[rt][0], b.x, b.y);
                        mma_bf16(part[rt][n], a[rt][1], b.z, b.w);
                    }
                }
            }
#pragma unroll
            for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    acc[rt][n][0] = fmaf(part[rt][n][0], sc[rt][0], acc[rt][n][0]);
                    acc[rt][n][1] = fmaf(part[rt][n][1], sc[rt][0], acc[rt][n][1]);
                    acc[rt][n][2] = fmaf(part[rt][n][2], sc[rt][1], acc[rt][n][2]);
                    acc[rt][n][3] = fmaf(part[rt][n][3], sc[rt][1], acc[rt][n][3]);
                }
        }
    }
    cp_async_wait<0>();
    __syncthreads(); /* the ring is dead; `red` may alias it */
#pragma unroll
    for (int rt = 0; rt < 2; ++rt)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            float *r0 = red + (size_t)(ks * kMmaRows + rt * 16 + g) * ldr + n * 8 + 2 * t;
            float *r1 = r0 + 8 * ldr;
            r0[0] = acc[rt][n][0]; r0[1] = acc[rt][n][1];
            r1[0] = acc[rt][n][2]; r1[1] = acc[rt][n][3];
        }
    __syncthreads();
}

template <int NT>
__global__ void __launch_bounds__(kMmaThreads) gate_up_mma_kernel(const MmaParams P, int stages) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int ldr = NT * 8 + 1;
    float *red = (float *)smem;
    const int row0 = blockIdx.x * 16; /* first gate/up pair of this CTA */
    if (blockIdx.x == 0 && threadIdx.x == 0 && P.tp_seq) atomicAdd(P.tp_seq, 1u); /* the call's number, read by the down launch */
    mma_block<NT, true>(P, row0, smem, stages, red, ldr);
    for (int i = threadIdx.x; i < 16 * P.M; i += kMmaThreads) {
        const int r = i % 16, m = i / 16;
        float gsum = 0.0f, usum = 0.0f;
#pragma unroll
        for (int ks = 0; ks < kMmaWarps; ++ks) {
            gsum += red[(size_t)(ks * kMmaRows + r) * ldr + m];
            usum += red[(size_t)(ks * kMmaRows + 16 + r) * ldr + m];
        }
        const uint16_t a = f32_to_bf16_bits(silu_mul(round_bf16(gsum), round_bf16(usum)));
        const int p = row0 + r;
        P.act[(size_t)m * P.up_offset + p] = a;
        P.act_perm[(size_t)m * P.up_offset + permute8(p)] = a;
    }
}

template <int NT>
__global__ void __launch_bounds__(kMmaThreads) down_mma_kernel(const MmaParams P, int stages) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int ldr = NT * 8 + 1;
    float *red = (float *)smem;
    const int row0 = blockIdx.x * kMmaRows;
    mma_block<NT, false>(P, row0, smem, stages, red, ldr);
    const unsigned seq = P.tp > 1 ? (*(volatile unsigned *)P.tp_seq - 1u) : 0u;
    const size_t slot = (size_t)((seq & 1u) * P.tp + P.rank) * P.slot_stride;
    for (int i = threadIdx.x; i < kMmaRows * P.M; i += kMmaThreads) {
        const int r = i % kMmaRows, m = i / kMmaRows;
        float y = 0.0f;
#pragma unroll
        for (int ks = 0; ks < kMmaWarps; ++ks) y += red[(size_t)(ks * kMmaRows + r) * ldr + m];
        const size_t o = (size_t)m * P.N + row0 + r;
        if (P.tp > 1) {
            for (int q = 0; q < P.tp; ++q) tp_store_tagged(P.peer_slots[q] + slot + o, y, seq + 1u);
        } else {
            const float v = round_bf16(y);
            P.out[o] = f32_to_bf16_bits(v);
            if (P.residual) P.residual[o] = f32_to_bf16_bits(bf16_bits_to_f32(P.residual[o]) + v);
        }
    }
    if (P.tp > 1) {
        /* every rank's partial sums of this CTA's rows arrive in this rank's own buffer as tagged
         * words: each thread waits (bounded) for the words of its own outputs and adds them in
         * rank order.  The thread stored its own words above, so no barrier is needed. */
        const unsigned long long *mine = P.peer_slots[P.rank] + (size_t)(seq & 1u) * P.tp * P.slot_stride;
        for (int i = threadIdx.x; i < kMmaRows * P.M; i += kMmaThreads) {
            const int r = i % kMmaRows, m = i / kMmaRows;
            const size_t o = (size_t)m * P.N + row0 + r;
            float y = 0.0f;
            bool all_in = true;
            for (int q = 0; q < P.tp && all_in; ++q) {
                const unsigned long long *p = mine + (size_t)q * P.slot_stride + o;
                float v = 0.0f;
                bool in = tp_load_tagged(p, seq + 1u, &v);
                for (uint32_t k = 0; !in && k < kTpPollLimit; ++k) {
                    __nanosleep(40);
                    in = tp_load_tagged(p, seq + 1u, &v);
                }
                all_in = in;
                y += v;
            }
            if (!all_in) { atomicCAS(P.status, 0u, 6u | ((unsigned)blockIdx.x << 8)); break; } /* 6 = peer data */
            const float v = round_bf16(y);
            P.out[o] = f32_to_bf16_bits(v);
            if (P.residual) P.residual[o] = f32_to_bf16_bits(bf16_bits_to_f32(P.residual[o]) + v);
        }
    }
}

/* x[m][k] -> xp[m][permute8(k)]: one thread moves one run of 8 */
__global__ void permute8_kernel(uint16_t *__restrict__ xp, const uint16_t *__restrict__ x, size_t runs) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= runs) return;
    const uint4 v = *(const uint4 *)(x + i * 8);
    const uint16_t *e = (const uint16_t *)&v;
    uint4 o;
    uint16_t *d = (uint16_t *)&o;
#pragma unroll
    for (int k = 0; k < 8; ++k) d[((k & 3) << 1) | (k >> 2)] = e[k];
    *(uint4 *)(xp + i * 8) = o;
}

/* ---- host ----------------------------------------------------------------------------------- */
static int mma_smem(int nt, int stages, int *stage_bytes_out) {
    const int xrow = kMmaKC * 2 + 64;
    const int stage = kMmaRows * kWRowBytes + nt * 8 * xrow;
    *stage_bytes_out = stage;
    const int red = kMmaWarps * kMmaRows * (nt * 8 + 1) * (int)sizeof(float);
    return max(stage * stages, red);
}

template <int NT>
static int launch_pair(const MmaParams &A, const MmaParams &B, int smem_optin, cudaStream_t stream) {
    int stage = 0;
    int stages = 4;
    while (stages > 2 && mma_smem(NT, stages, &stage) > smem_optin) --stages;
    const int smem = mma_smem(NT, stages, &stage);
    if (smem > smem_optin) return fail(FFN_ERR_CONFIG, "batched INT4 FFN: %d tokens do not fit shared memory", NT * 8);
    FFN_CUDA_TRY(cudaFuncSetAttribute(gate_up_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "gate/up MMA: shared-memory opt-in");
    FFN_CUDA_TRY(cudaFuncSetAttribute(down_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "down MMA: shared-memory opt-in");
    gate_up_mma_kernel<NT><<<A.up_offset / 16, kMmaThreads, smem, stream>>>(A, stages);
    FFN_CUDA_TRY(cudaGetLastError(), "gate/up MMA launch");
    down_mma_kernel<NT><<<B.N / kMmaRows, kMmaThreads, smem, stream>>>(B, stages);
    FFN_CUDA_TRY(cudaGetLastError(), "down MMA launch");
    return FFN_OK;
}

/* Per device: room for the permuted copies of the input and of act (bf16 [tokens][H + I]).  Grown on
 * demand, so the first call of a new size allocates (make it before capturing a graph). */
static void *g_mma_scratch[64];
static size_t g_mma_scratch_bytes[64];

/* normed bf16 [tokens][H] -> layer_out bf16 [tokens][H]; `act` receives act in natural order. */
int mma_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                   const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual, unsigned *status) {
    if (tokens < 1 || tokens > 64) return FFN_NOT_ADMITTED;
    if (H % kMmaRows || I % 16) return FFN_NOT_ADMITTED;
    if (((uintptr_t)w->gate_up_i4 & 15) || ((uintptr_t)w->down_i4 & 15) || ((uintptr_t)normed & 15))
        return FFN_NOT_ADMITTED;
    int dev = 0, smem_optin = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FFN_ERR_CONFIG, "device index %d out of range", dev);
    FFN_CUDA_TRY(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "smem opt-in");
    const size_t need = (size_t)tokens * (H + I) * sizeof(uint16_t);
    if (g_mma_scratch_bytes[dev] < need) {
        const size_t want = (size_t)64 * (H + I) * sizeof(uint16_t); /* the largest batch this path takes */
        if (g_mma_scratch[dev]) { FFN_CUDA_TRY(cudaDeviceSynchronize(), "batched INT4 FFN: scratch regrow"); cudaFree(g_mma_scratch[dev]); }
        g_mma_scratch[dev] = nullptr; g_mma_scratch_bytes[dev] = 0;
        if (cudaMalloc(&g_mma_scratch[dev], want) != cudaSuccess) { (void)cudaGetLastError(); return fail(FFN_ERR_ALLOC, "batched INT4 FFN: cannot allocate %zu bytes of scratch", want); }
        g_mma_scratch_bytes[dev] = want;
    }
    uint16_t *xp = (uint16_t *)g_mma_scratch[dev];
    uint16_t *act_perm = xp + (size_t)tokens * H;
    const size_t runs = (size_t)tokens * H / 8;
    permute8_kernel<<<(unsigned)((runs + 255) / 256), 256, 0, stream>>>(xp, (const uint16_t *)normed, runs);
    FFN_CUDA_TRY(cudaGetLastError(), "permute launch");

    MmaParams A = {};
    A.x = xp; A.w = w->gate_up_i4; A.s = (const uint16_t *)w->gate_up_i4_scales;
    A.M = tokens; A.N = 2 * I; A.K = H; A.up_offset = I;
    A.act = (uint16_t *)act; A.act_perm = act_perm;
    A.tp = 1; A.status = status;
    MmaParams B = {};
    B.x = act_perm; B.w = w->down_i4; B.s = (const uint16_t *)w->down_i4_scales;
    B.M = tokens; B.N = H; B.K = I; B.up_offset = 0;
    B.out = (uint16_t *)layer_out; B.residual = (uint16_t *)residual;
    B.tp = 1; B.status = status;
    if (tp && tp->tp > 1) {
        if (tokens * H > tp->slot_stride) return fail(FFN_ERR_CONFIG, "batched INT4 FFN: %d tokens exceed the exchange buffer", tokens);
        A.tp_seq = tp->seq;
        B.tp = tp->tp; B.rank = tp->rank; B.slot_stride = tp->slot_stride;
        B.peer_slots = tp->peer_slots; B.tp_seq = tp->seq;
    }
    if (tokens <= 8) return launch_pair<1>(A, B, smem_optin, stream);
    if (tokens <= 16) return launch_pair<2>(A, B, smem_optin, stream);
    if (tokens <= 32) return launch_pair<4>(A, B, smem_optin, stream);
    return launch_pair<8>(A, B, smem_optin, stream);
}

}  // namespace ffn
