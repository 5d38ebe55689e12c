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
 * the next launch), then down with the cross-rank exchange in its epilogue (the tagged-word protocol
 * of the fused decode kernel).  A CTA takes 128 weight rows (64 gate + 64 up, or 128 down rows), one
 * 16-row MMA tile per warp, so every activation byte it brings into shared memory is used by 128
 * rows.  The down projection has only H/128 row blocks, so its K range is split over several CTAs
 * per block; each writes FP32 partial sums to global memory and the last one to arrive adds them in
 * split order (deterministic) and runs the epilogue.
 */
#include <stdio.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace ffn {

constexpr int kMmaWarps = 8;          /* one 16-row MMA tile each, every group of the K chunk */
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaRows = 16 * kMmaWarps; /* 128 weight rows per CTA: the activations a CTA loads are reused 128 times */
constexpr int kMmaKC = 256;           /* K per pipeline stage: 2 groups */
constexpr int kMmaGroupsPerChunk = kMmaKC / FFN_INT4_GROUP;
constexpr int kWRowBytes = kMmaKC / 2 + 16;   /* 144: conflict-free 32-bit reads down 8 rows */
constexpr int kMmaMaxSplits = 8;      /* K splits of the down projection (partial sums through global memory) */

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
    /* down: K split over `splits` CTAs per row block */
    int splits;
    float *partial;           /* [splits][M][N] fp32 */
    unsigned *arrivals;       /* [N / kMmaRows], zero between launches */
    /* tensor parallelism (down only) */
    int tp, rank, slot_stride;
    unsigned long long *const *peer_slots;
    unsigned *tp_seq;
    unsigned *status;         /* word 3 of the device's synchronisation words */
};

/* One CTA: 128 weight rows ([gate64 | up64] or down128) x all tokens over the groups [gbeg, gend) of
 * K, streamed in 256-wide chunks through a cp.async ring; warp wp owns rows 16*wp .. 16*wp+15.  On
 * return red[row * ldr + token] holds the FP32 sums. */
template <int NT, bool PAIRS>
__device__ __forceinline__ void mma_block(const MmaParams &P, int row0, int gbeg, int gend, uint8_t *smem, int stages,
                                          float *red, int ldr) {
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr int xrow = kMmaKC * 2 + 64;                 /* bytes per token row of a stage, = 64 mod 128 */
    constexpr int stage_bytes = kMmaRows * kWRowBytes + NT * 8 * xrow;
    const int G = P.K / FFN_INT4_GROUP;
    const int ngroups = gend - gbeg;
    const int nchunks = (ngroups + kMmaGroupsPerChunk - 1) / kMmaGroupsPerChunk;
    const uint32_t sbase = smem_addr(smem);

    auto row_of = [&](int r) -> int { /* global weight row of local row r */
        return PAIRS ? (r < kMmaRows / 2 ? row0 + r : P.up_offset + row0 + (r - kMmaRows / 2)) : row0 + r;
    };
    /* Each thread copies the same pieces of every chunk: 4 weight pieces (row r = i/8, 16-byte column
     * c = i%8) and NT activation pieces (token m = i/32, column c = i%32).  Sources and shared
     * offsets are fixed per thread, so a chunk costs one add per piece. */
    const uint8_t *wsrc[4];
    uint32_t wdst[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int i = tid + q * kMmaThreads, r = i >> 3, c = i & 7;
        wsrc[q] = P.w + (size_t)row_of(r) * (P.K / 2) + (size_t)gbeg * (FFN_INT4_GROUP / 2) + c * 16;
        wdst[q] = (uint32_t)(r * kWRowBytes + c * 16);
    }
    const uint16_t *xsrc[NT];
    uint32_t xdst[NT];
#pragma unroll
    for (int q = 0; q < NT; ++q) {
        const int i = tid + q * kMmaThreads, m = i >> 5, c = i & 31;
        xsrc[q] = m < P.M ? P.x + (size_t)m * P.K + (size_t)gbeg * FFN_INT4_GROUP + c * 8 : nullptr;
        xdst[q] = (uint32_t)(kMmaRows * kWRowBytes + m * xrow + c * 16);
    }
    const int tcol_w = (tid & 7) * 32, tcol_x = (tid & 31) * 8; /* first K index (in the chunk) of this thread's pieces */
    auto issue = [&](int chunk) {
        const uint32_t st = sbase + (uint32_t)(chunk % stages) * stage_bytes;
        const int k0 = chunk * kMmaKC, kc = min(kMmaKC, ngroups * FFN_INT4_GROUP - k0);
        if (tcol_w < kc) {
#pragma unroll
            for (int q = 0; q < 4; ++q) cp_async16(st + wdst[q], wsrc[q] + k0 / 2);
        }
        if (tcol_x < kc) {
#pragma unroll
            for (int q = 0; q < NT; ++q)
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

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    const int r_lo = row_of(wp * 16 + g), r_hi = row_of(wp * 16 + g + 8);
    const uint16_t *s_lo = P.s + (size_t)r_lo * G + gbeg, *s_hi = P.s + (size_t)r_hi * G + gbeg;

    for (int c = 0; c < stages - 1; ++c) {
        if (c < nchunks) issue(c); else cp_async_commit();
    }
    for (int c = 0; c < nchunks; ++c) {
        /* chunk c was committed `stages - 1` groups ago: all but the newest stages-2 groups must be done */
        if (stages == 4) cp_async_wait<2>(); else if (stages == 3) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads(); /* everyone sees chunk c, and everyone is done with the buffer refilled below */
        if (c + stages - 1 < nchunks) issue(c + stages - 1); else cp_async_commit();
        const uint32_t st = sbase + (uint32_t)(c % stages) * stage_bytes;
#pragma unroll
        for (int gi = 0; gi < kMmaGroupsPerChunk; ++gi) {
            const int grp = c * kMmaGroupsPerChunk + gi; /* relative to gbeg */
            if (grp < ngroups) {
                const float sc_lo = bf16_bits_to_f32(__ldg(s_lo + grp)), sc_hi = bf16_bits_to_f32(__ldg(s_hi + grp));
                const uint32_t xs = st + kMmaRows * kWRowBytes + (uint32_t)g * xrow + (uint32_t)gi * 256;
                const uint32_t wa0 = st + (uint32_t)(wp * 16 + g) * kWRowBytes + (uint32_t)gi * 64 + (uint32_t)t * 4;
                float part[NT][4];
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) part[n][i] = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t a[2][4]; /* [mma of the pair][a0..a3] */
                    const uint32_t w_lo = lds32(wa0 + (uint32_t)j * 16), w_hi = lds32(wa0 + (uint32_t)j * 16 + 8 * kWRowBytes); /* rows g, g+8 */
                    a[0][0] = codes_bf16x2(w_lo, 0); a[0][1] = codes_bf16x2(w_hi, 0);
                    a[0][2] = codes_bf16x2(w_lo, 1); a[0][3] = codes_bf16x2(w_hi, 1);
                    a[1][0] = codes_bf16x2(w_lo, 2); a[1][1] = codes_bf16x2(w_hi, 2);
                    a[1][2] = codes_bf16x2(w_lo, 3); a[1][3] = codes_bf16x2(w_hi, 3);
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        const uint4 b = lds128(xs + (uint32_t)n * 8 * xrow + (uint32_t)(4 * j + t) * 16);
                        mma_bf16(part[n], a[0], b.x, b.y);
                        mma_bf16(part[n], a[1], b.z, b.w);
                    }
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    acc[n][0] = fmaf(part[n][0], sc_lo, acc[n][0]);
                    acc[n][1] = fmaf(part[n][1], sc_lo, acc[n][1]);
                    acc[n][2] = fmaf(part[n][2], sc_hi, acc[n][2]);
                    acc[n][3] = fmaf(part[n][3], sc_hi, acc[n][3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads(); /* the ring is dead; `red` may alias it */
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        float *r0 = red + (size_t)(wp * 16 + g) * ldr + n * 8 + 2 * t;
        float *r1 = r0 + 8 * ldr;
        r0[0] = acc[n][0]; r0[1] = acc[n][1];
        r1[0] = acc[n][2]; r1[1] = acc[n][3];
    }
    __syncthreads();
}

template <int NT>
__global__ void __launch_bounds__(kMmaThreads) gate_up_mma_kernel(const MmaParams P, int stages) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int ldr = NT * 8 + 1;
    float *red = (float *)smem;
    constexpr int kPairs = kMmaRows / 2;
    const int row0 = blockIdx.x * kPairs; /* first gate/up pair of this CTA */
    if (blockIdx.x == 0 && threadIdx.x == 0 && P.tp_seq) atomicAdd(P.tp_seq, 1u); /* the call's number, read by the down launch */
    mma_block<NT, true>(P, row0, 0, P.K / FFN_INT4_GROUP, smem, stages, red, ldr);
    for (int i = threadIdx.x; i < kPairs * P.M; i += kMmaThreads) {
        const int r = i % kPairs, m = i / kPairs;
        const float gsum = red[(size_t)r * ldr + m], usum = red[(size_t)(kPairs + r) * ldr + m];
        const uint16_t a = f32_to_bf16_bits(silu_mul(round_bf16(gsum), round_bf16(usum)));
        const int p = row0 + r;
        P.act[(size_t)m * P.up_offset + p] = a;
        P.act_perm[(size_t)m * P.up_offset + permute8(p)] = a;
    }
}

template <int NT>
__global__ void __launch_bounds__(kMmaThreads) down_mma_kernel(const MmaParams P, int stages) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int last_arrival;
    const int ldr = NT * 8 + 1;
    float *red = (float *)smem;
    const int rb = blockIdx.x / P.splits, sp = blockIdx.x % P.splits;
    const int row0 = rb * kMmaRows;
    const int G = P.K / FFN_INT4_GROUP;
    mma_block<NT, false>(P, row0, (int)((long long)G * sp / P.splits), (int)((long long)G * (sp + 1) / P.splits), smem, stages, red, ldr);
    if (P.splits > 1) {
        /* this CTA's share of K is done: leave it in global memory; whoever arrives last at the row
         * block adds the shares in split order and carries on alone */
        for (int i = threadIdx.x; i < kMmaRows * P.M; i += kMmaThreads) {
            const int r = i % kMmaRows, m = i / kMmaRows;
            __stcg(P.partial + ((size_t)sp * P.M + m) * P.N + row0 + r, red[(size_t)r * ldr + m]);
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned before = atomicAdd(P.arrivals + rb, 1u);
            last_arrival = before == (unsigned)P.splits - 1u;
            if (last_arrival) P.arrivals[rb] = 0u; /* ready for the next launch */
        }
        __syncthreads();
        if (!last_arrival) return;
        __threadfence();
        /* every load of an element is issued before the first add, and four elements go together: a loop
         * of load-then-add over a run-time split count serialises the trips to L2 (224 of them per
         * thread at 64 tokens).  Measured against a split-outer form with eight elements in flight:
         * this one is the faster (185.6 vs 204.0 us per FFN at 64 tokens, 72.5 vs 74.5 at 16). */
#pragma unroll 4
        for (int i = threadIdx.x; i < kMmaRows * P.M; i += kMmaThreads) {
            const int r = i % kMmaRows, m = i / kMmaRows;
            float v[kMmaMaxSplits];
#pragma unroll
            for (int q = 0; q < kMmaMaxSplits; ++q)
                v[q] = q < P.splits ? __ldcg(P.partial + ((size_t)q * P.M + m) * P.N + row0 + r) : 0.0f;
            float y = 0.0f;
#pragma unroll
            for (int q = 0; q < kMmaMaxSplits; ++q)
                if (q < P.splits) y += v[q];
            red[(size_t)r * ldr + m] = y;
        }
        /* each thread reads back only what it wrote to `red` itself: no barrier needed */
    }
    const unsigned seq = P.tp > 1 ? (*(volatile unsigned *)P.tp_seq - 1u) : 0u;
    const size_t slot = (size_t)((seq & 1u) * P.tp + P.rank) * P.slot_stride;
    for (int i = threadIdx.x; i < kMmaRows * P.M; i += kMmaThreads) {
        const int r = i % kMmaRows, m = i / kMmaRows;
        const float y = red[(size_t)r * ldr + m];
        const size_t o = (size_t)m * P.N + row0 + r;
        if (P.tp > 1) {
            for (int q = 0; q < P.tp; ++q) tp_store_tagged(P.peer_slots[q] + slot + o, y, tp_tag(seq));
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
            const bool all_in = tp_wait_sum(mine + o, (size_t)P.slot_stride, P.tp, tp_tag(seq), nullptr, 40, &y);
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
static int mma_stage_bytes(int nt) { return kMmaRows * kWRowBytes + nt * 8 * (kMmaKC * 2 + 64); }
static int mma_smem(int nt, int stages) {
    const int red = kMmaRows * (nt * 8 + 1) * (int)sizeof(float);
    return max(mma_stage_bytes(nt) * stages, red);
}

/* Per device: the permuted copies of the input and of act (bf16 [tokens][H + I]), the split-K partial
 * sums of the down projection and its arrival counters.  Grown on demand, so the first call of a new
 * size allocates (make it before capturing a graph). */
struct MmaScratch {
    uint8_t *base = nullptr;
    size_t bytes = 0;
};
static MmaScratch g_mma_scratch[64];
static std::mutex g_mma_mutex; /* guards the table above; the scratch itself is shared by every call on the device */

/* Launch geometry of the pair for `nt` 8-token tiles: pipeline depth, shared memory per CTA, CTAs per
 * SM, and the K splits of the down projection (chosen to fill the device's CTA slots as evenly as
 * possible).  Needs no device.  Returns false when the tokens do not fit shared memory. */
struct MmaPlan {
    int stages, smem, per_sm, splits, gate_up_ctas, down_ctas;
};
static bool mma_plan(int nt, int H, int I, int smem_optin, int sm_count, MmaPlan &pl) {
    /* four stages when two CTAs still fit on an SM, else three if that makes two fit, else four */
    int stages = 4;
    if (2 * (mma_smem(nt, 4) + 1024) > smem_optin && 2 * (mma_smem(nt, 3) + 1024) <= smem_optin) stages = 3;
    while (stages > 2 && mma_smem(nt, stages) > smem_optin) --stages;
    const int smem = mma_smem(nt, stages);
    if (smem > smem_optin) return false;
    const int per_sm = 2 * (smem + 1024) <= smem_optin ? 2 : 1;
    const int blocks = H / kMmaRows, slots = sm_count * per_sm, G = I / FFN_INT4_GROUP;
    int best = 1;
    double best_eff = 0.0;
    for (int sp = 1; sp <= kMmaMaxSplits && sp * 2 <= max(G, 2); ++sp) {
        const int units = blocks * sp;
        const double eff = (double)units / (double)(((units + slots - 1) / slots) * slots);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = sp; }
    }
    pl.stages = stages; pl.smem = smem; pl.per_sm = per_sm; pl.splits = best;
    pl.gate_up_ctas = I / (kMmaRows / 2); pl.down_ctas = blocks * best;
    return true;
}

template <int NT>
static int launch_pair(MmaParams &A, MmaParams &B, int smem_optin, int sm_count, cudaStream_t stream) {
    MmaPlan pl;
    if (!mma_plan(NT, B.N, B.K, smem_optin, sm_count, pl))
        return fail(FFN_ERR_CONFIG, "batched INT4 FFN: %d tokens do not fit shared memory", NT * 8);
    const int stages = pl.stages, smem = pl.smem, blocks = B.N / kMmaRows;
    B.splits = pl.splits;
    FFN_CUDA_TRY(cudaFuncSetAttribute(gate_up_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "gate/up MMA: shared-memory opt-in");
    FFN_CUDA_TRY(cudaFuncSetAttribute(down_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "down MMA: shared-memory opt-in");
    gate_up_mma_kernel<NT><<<A.up_offset / (kMmaRows / 2), kMmaThreads, smem, stream>>>(A, stages);
    FFN_CUDA_TRY(cudaGetLastError(), "gate/up MMA launch");
    down_mma_kernel<NT><<<blocks * B.splits, kMmaThreads, smem, stream>>>(B, stages);
    FFN_CUDA_TRY(cudaGetLastError(), "down MMA launch");
    return FFN_OK;
}

static int mma_tiles_for(int tokens) { return tokens <= 8 ? 1 : tokens <= 16 ? 2 : tokens <= 32 ? 4 : 8; }

bool mma_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes) {
    if (tokens < 1 || tokens > 64 || H <= 0 || I <= 0 || H % kMmaRows || I % (kMmaRows / 2) || I % FFN_INT4_GROUP) return false;
    MmaPlan pl;
    const int nt = mma_tiles_for(tokens);
    if (!mma_plan(nt, H, I, smem_optin, sm_count, pl)) return false;
    snprintf(out, out_bytes,
             "kernel=mma_pair token_tiles=%d threads=%d smem=%d stages=%d ctas_per_sm=%d gate_up_ctas=%d down_ctas=%d down_k_splits=%d",
             nt, kMmaThreads, pl.smem, pl.stages, pl.per_sm, pl.gate_up_ctas, pl.down_ctas, pl.splits);
    return true;
}

/* normed bf16 [tokens][H] -> layer_out bf16 [tokens][H]; `act` receives act in natural order. */
int mma_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                   const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual, unsigned *status) {
    if (tokens < 1 || tokens > 64) return FFN_NOT_ADMITTED;
    if (H % kMmaRows || I % (kMmaRows / 2)) return FFN_NOT_ADMITTED;
    if (((uintptr_t)w->gate_up_i4 & 15) || ((uintptr_t)w->down_i4 & 15) || ((uintptr_t)normed & 15))
        return FFN_NOT_ADMITTED;
    int dev = 0, smem_optin = 0, sm_count = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FFN_ERR_CONFIG, "device index %d out of range", dev);
    FFN_CUDA_TRY(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "smem opt-in");
    FFN_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev), "SM count");
    /* layout: [arrival counters 4 KiB | x permuted | act permuted | partial sums], sized for 64 tokens */
    const size_t counters = 4096;
    if ((size_t)(H / kMmaRows) * sizeof(unsigned) > counters) return FFN_NOT_ADMITTED;
    const size_t perm_bytes = ((size_t)64 * (H + I) * sizeof(uint16_t) + 255) / 256 * 256;
    const size_t want = counters + perm_bytes + (size_t)kMmaMaxSplits * 64 * H * sizeof(float);
    std::lock_guard<std::mutex> lock(g_mma_mutex);
    MmaScratch &sc = g_mma_scratch[dev];
    if (sc.bytes < want) {
        if (sc.base) { FFN_CUDA_TRY(cudaDeviceSynchronize(), "batched INT4 FFN: scratch regrow"); cudaFree(sc.base); }
        sc.base = nullptr; sc.bytes = 0;
        if (cudaMalloc(&sc.base, want) != cudaSuccess) { (void)cudaGetLastError(); return fail(FFN_ERR_ALLOC, "batched INT4 FFN: cannot allocate %zu bytes of scratch", want); }
        FFN_CUDA_TRY(cudaMemset(sc.base, 0, counters), "batched INT4 FFN: clear arrival counters");
        sc.bytes = want;
    }
    uint16_t *xp = (uint16_t *)(sc.base + counters);
    uint16_t *act_perm = xp + (size_t)tokens * H;
    const size_t runs = (size_t)tokens * H / 8;
    permute8_kernel<<<(unsigned)((runs + 255) / 256), 256, 0, stream>>>(xp, (const uint16_t *)normed, runs);
    FFN_CUDA_TRY(cudaGetLastError(), "permute launch");

    MmaParams A = {};
    A.x = xp; A.w = w->gate_up_i4; A.s = (const uint16_t *)w->gate_up_i4_scales;
    A.M = tokens; A.N = 2 * I; A.K = H; A.up_offset = I;
    A.act = (uint16_t *)act; A.act_perm = act_perm;
    A.tp = 1; A.status = status; A.splits = 1;
    MmaParams B = {};
    B.x = act_perm; B.w = w->down_i4; B.s = (const uint16_t *)w->down_i4_scales;
    B.M = tokens; B.N = H; B.K = I; B.up_offset = 0;
    B.out = (uint16_t *)layer_out; B.residual = (uint16_t *)residual;
    B.tp = 1; B.status = status; B.splits = 1;
    B.partial = (float *)(sc.base + counters + perm_bytes);
    B.arrivals = (unsigned *)sc.base;
    if (tp && tp->tp > 1) {
        if (tokens * H > tp->slot_stride) return fail(FFN_ERR_CONFIG, "batched INT4 FFN: %d tokens exceed the exchange buffer", tokens);
        A.tp_seq = tp->seq;
        B.tp = tp->tp; B.rank = tp->rank; B.slot_stride = tp->slot_stride;
        B.peer_slots = tp->peer_slots; B.tp_seq = tp->seq;
    }
    switch (mma_tiles_for(tokens)) {
        case 1: return launch_pair<1>(A, B, smem_optin, sm_count, stream);
        case 2: return launch_pair<2>(A, B, smem_optin, sm_count, stream);
        case 4: return launch_pair<4>(A, B, smem_optin, sm_count, stream);
        default: return launch_pair<8>(A, B, smem_optin, sm_count, stream);
    }
}

}  // namespace ffn
