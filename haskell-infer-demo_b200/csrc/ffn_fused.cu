/*
 * ffn_fused.cu - the decode-shaped (M <= 2) INT4 FFN as ONE persistent kernel per call:
 *
 *     act = bf16( silu(bf16(W_gate x)) * bf16(W_up x) )      phase 1, column-parallel rows
 *     y   = bf16( sum over ranks of W_down[:, slice] act )   phase 2, row-parallel, fused reduce
 *
 * replacing the reference's three launches per rank (gemv_int4_kernel, silu_mul_packed_kernel,
 * gemv_int4_kernel; csrc/kernels/layers.cu:127-145) and, under tensor parallelism, the host-issued
 * leader all-reduce that follows them (csrc/collective.cu:168-219; csrc/engine.cu:1436-1452).
 *
 * Shape of the kernel (one CTA per SM, 19 warps):
 *   warp 0        producer: streams this CTA's contiguous share of the packed weight rows from HBM
 *                 into a shared-memory ring with cp.async.bulk, completion counted on mbarriers.
 *                 The stream does not stop at the phase boundary: down-projection rows are already
 *                 in flight while the grid waits for the activation vector.
 *   warps 1..17   consumers: thread (ct, rg) owns 16-byte column chunk(s) ct of every row r with
 *                 r % RG == rg of a tile.  Its slice of the activation vector lives in registers
 *                 for the whole phase; weights are unpacked from shared memory and multiplied with
 *                 BF16 x FP32-accumulate FMAs; half-warp shuffles reduce the row partials.
 *   warp 18       epilogue: adds the half-warp partials in a fixed order (deterministic), applies
 *                 the reference's rounding points, stores act / y, runs the grid barrier arrival and
 *                 the cross-GPU exchange.
 *
 * Cross-rank reduce (TP = R > 1): CTA c of every rank owns the same output rows.  Its epilogue
 * stores the FP32 partials of those rows into slot `rank` of a [2][R][M][H] buffer in EVERY rank's
 * memory (plain peer stores over NVLink), publishes them with a system-scope release increment of
 * flag[c] on every rank, waits (bounded) until its own flag[c] shows all R arrivals, then adds the R
 * slots in rank order and rounds once to BF16.  No collective call and no second kernel.
 *
 * Every device-side wait is bounded; on expiry the kernel records where it gave up in the status
 * word, drains its own copies and returns.  The host maps that to FFN_ERR_CUDA.
 */
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace ffn {

constexpr int kConsumerWarps = 17;
constexpr int kConsumerThreads = kConsumerWarps * 32;  /* 544 = 17 * 32: I = 17408 = 17 * 1024 */
constexpr int kEpilogueWarp = kConsumerWarps + 1;
constexpr int kThreads = (kConsumerWarps + 2) * 32;    /* 608 */
constexpr int kMaxStages = 8;
constexpr int kPartSlots = 4;
constexpr int kPartFloats = 512;                       /* floats per partial slot */
constexpr int kMaxJT = 4;                              /* row steps per thread per tile */
constexpr uint32_t kSpinLimit = 1u << 24;              /* bounded waits: ~1 s worst case */

/* status word values (where a wait gave up) */
enum { ST_OK = 0, ST_PRODUCER_EMPTY = 1, ST_CONSUMER_FULL = 2, ST_PART_EMPTY = 3, ST_PART_FULL = 4,
       ST_GRID_BARRIER = 5, ST_PEER_FLAG = 6, ST_DRAIN = 7 };

struct PhasePlan {
    const uint8_t *w;     /* packed rows */
    const uint16_t *s;    /* scales */
    int K, rb, cpr, G;    /* columns, row bytes, 16-byte chunks per row, groups per row */
    int CT, RG, JT, TR;   /* column threads, row groups, row steps per tile, rows(pairs) per tile */
    int rows_total;       /* rows (phase 2) or gate/up pairs (phase 1) this rank owns */
    int up_offset;        /* phase 1: row index of up row 0 (= local I) */
    int nhw;              /* half-warps per row group = CT / 16 */
};

struct FusedParams {
    const uint16_t *x;    /* [M][H] bf16 */
    uint16_t *act;        /* [M][I] bf16 (global scratch the caller's workspace provides) */
    uint16_t *out;        /* [M][H] bf16 */
    PhasePlan p1, p2;
    int M, H, I;
    int stage_bytes, nstages;
    unsigned *sync;       /* [0] arrival count, [1] generation, [2] call sequence, [3] status */
    /* tensor parallelism (tp == 1: unused) */
    int tp, rank;
    float *const *peer_slots;   /* device array [tp]: each rank's [2][tp][M_max][H] fp32 slots */
    unsigned *const *peer_flags;/* device array [tp]: each rank's per-CTA arrival counters */
    int slot_stride;      /* floats per (parity, rank) slot = M_max * H */
    /* optional fused residual update on the reduced output (h <- bf16(h + y)); NULL = off */
    uint16_t *residual;
};

/* ---- PTX wrappers -------------------------------------------------------------------------- */
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
/* Bounded wait.  Returns false when the limit ran out or another thread already gave up. */
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint4 lds16(const void *p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ uint4 ldg_cg16(const void *p) { /* coherent at L2: data other CTAs just wrote */
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned *p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float *p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

/* ---- the inner product of one 16-byte chunk (32 codes) with 32 BF16 activations ------------- */
/* (w & 0x000F000F) ^ 0x43084308 puts, in each 16-bit half, the BF16 value 128 + (code + 8): the
 * nibble XOR 8 is code+8 in [1,15] and sits in the low mantissa bits of 128.0 (0x4300).  The
 * mixed-precision FMA multiplies that BF16 by the BF16 activation exactly and accumulates in FP32,
 * so one logic op converts two codes and no integer-to-float conversion is issued.  The constant
 * 136 * sum(x) is removed once per chunk (xoff): sum((136 + c_k) x_k) - 136 sum(x_k) = sum(c_k x_k). */
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); /* (a & b) ^ c */
    return d;
}
__device__ __forceinline__ float fma_bf16_lo_lo(uint32_t a, uint32_t b, float c) {
    float d;
    asm("{\n.reg .b16 al, ah, bl, bh;\nmov.b32 {al, ah}, %1;\nmov.b32 {bl, bh}, %2;\nfma.rn.f32.bf16 %0, al, bl, %3;\n}"
        : "=f"(d) : "r"(a), "r"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fma_bf16_lo_hi(uint32_t a, uint32_t b, float c) {
    float d;
    asm("{\n.reg .b16 al, ah, bl, bh;\nmov.b32 {al, ah}, %1;\nmov.b32 {bl, bh}, %2;\nfma.rn.f32.bf16 %0, al, bh, %3;\n}"
        : "=f"(d) : "r"(a), "r"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fma_bf16_hi_lo(uint32_t a, uint32_t b, float c) {
    float d;
    asm("{\n.reg .b16 al, ah, bl, bh;\nmov.b32 {al, ah}, %1;\nmov.b32 {bl, bh}, %2;\nfma.rn.f32.bf16 %0, ah, bl, %3;\n}"
        : "=f"(d) : "r"(a), "r"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fma_bf16_hi_hi(uint32_t a, uint32_t b, float c) {
    float d;
    asm("{\n.reg .b16 al, ah, bl, bh;\nmov.b32 {al, ah}, %1;\nmov.b32 {bl, bh}, %2;\nfma.rn.f32.bf16 %0, ah, bh, %3;\n}"
        : "=f"(d) : "r"(a), "r"(b), "f"(c));
    return d;
}

/* One 32-bit word (codes k = 8j .. 8j+7) against x pairs xr[0..3] = {x0,x1},{x2,x3},{x4,x5},{x6,x7}.
 * MT tokens share the converted weights. */
template <int MT>
__device__ __forceinline__ void word_dot(uint32_t w, const uint32_t (*xr)[16], int j, float (&acc)[MT]) {
    const uint32_t v0 = lop3_and_xor(w, 0x000F000Fu, 0x43084308u);       /* k = 0 (lo), 4 (hi) */
    const uint32_t v1 = lop3_and_xor(w >> 4, 0x000F000Fu, 0x43084308u);  /* k = 1, 5 */
    const uint32_t v2 = lop3_and_xor(w >> 8, 0x000F000Fu, 0x43084308u);  /* k = 2, 6 */
    const uint32_t v3 = lop3_and_xor(w >> 12, 0x000F000Fu, 0x43084308u); /* k = 3, 7 */
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint32_t *x = xr[m] + 4 * j;
        float a = acc[m];
        a = fma_bf16_lo_lo(v0, x[0], a);
        a = fma_bf16_lo_hi(v1, x[0], a);
        a = fma_bf16_lo_lo(v2, x[1], a);
        a = fma_bf16_lo_hi(v3, x[1], a);
        a = fma_bf16_hi_lo(v0, x[2], a);
        a = fma_bf16_hi_hi(v1, x[2], a);
        a = fma_bf16_hi_lo(v2, x[3], a);
        a = fma_bf16_hi_hi(v3, x[3], a);
        acc[m] = a;
    }
}

template <int MT>
__device__ __forceinline__ void chunk_dot(const uint4 &w, const uint32_t (*xr)[16], float (&acc)[MT]) {
    word_dot<MT>(w.x, xr, 0, acc);
    word_dot<MT>(w.y, xr, 1, acc);
    word_dot<MT>(w.z, xr, 2, acc);
    word_dot<MT>(w.w, xr, 3, acc);
}

/* Sum of NV values over the 16 lanes of a half-warp; value i ends up in lane (16/NV)*i of the
 * half-warp (and its NV-1.. neighbours).  NV in {1, 2, 4}. */
template <int NV>
__device__ __forceinline__ float halfwarp_reduce(float (&v)[NV], int lane, unsigned mask) {
    float r;
    if (NV == 4) {
        const bool b8 = lane & 8;
        float k0 = b8 ? v[2] : v[0], k1 = b8 ? v[3] : v[1];
        const float s0 = b8 ? v[0] : v[2], s1 = b8 ? v[1] : v[3];
        k0 += __shfl_xor_sync(mask, s0, 8);
        k1 += __shfl_xor_sync(mask, s1, 8);
        const bool b4 = lane & 4;
        r = b4 ? k1 : k0;
        const float s = b4 ? k0 : k1;
        r += __shfl_xor_sync(mask, s, 4);
        r += __shfl_xor_sync(mask, r, 2);
        r += __shfl_xor_sync(mask, r, 1);
    } else if (NV == 2) {
        const bool b8 = lane & 8;
        r = b8 ? v[1] : v[0];
        const float s = b8 ? v[0] : v[1];
        r += __shfl_xor_sync(mask, s, 8);
        r += __shfl_xor_sync(mask, r, 4);
        r += __shfl_xor_sync(mask, r, 2);
        r += __shfl_xor_sync(mask, r, 1);
    } else {
        r = v[0];
        r += __shfl_xor_sync(mask, r, 8);
        r += __shfl_xor_sync(mask, r, 4);
        r += __shfl_xor_sync(mask, r, 2);
        r += __shfl_xor_sync(mask, r, 1);
    }
    return r;
}

struct Smem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t part_full[kPartSlots];
    uint64_t part_empty[kPartSlots];
    int abort_flag;
    int pad[15];
    float part[kPartSlots][kPartFloats];
};

__device__ __forceinline__ void give_up(Smem *sm, unsigned *sync, int where) {
    sm->abort_flag = 1;
    atomicCAS(sync + 3, 0u, (unsigned)where | ((unsigned)blockIdx.x << 8));
}

__device__ __forceinline__ int cta_begin(int total, int cta, int ctas) {
    return (int)(((long long)total * cta) / ctas);
}

/* ---- consumer side of one phase ------------------------------------------------------------ */
template <int CIT, int MT, bool PAIRS>
__device__ __forceinline__ void consume_phase(const PhasePlan &pl, const uint16_t *xsrc, Smem *sm,
                                              uint8_t *ring, int stage_bytes, int nstages, int tile0,
                                              unsigned *sync) {
    constexpr int NVROW = (PAIRS ? 2 : 1) * MT;
    constexpr int JTM = PAIRS ? 1 : kMaxJT; /* phase 1 tiles hold one pair per row group */
    const int ti = threadIdx.x - 32;
    const int lane = threadIdx.x & 31;
    const int warp_lane0 = lane == 0;
    const bool active = ti < pl.CT * pl.RG;
    const int ct = ti % pl.CT, rg = ti / pl.CT;
    const unsigned hmask = 0xFFFFu << (lane & 16);
    const int row_begin = cta_begin(pl.rows_total, blockIdx.x, gridDim.x);
    const int row_end = cta_begin(pl.rows_total, blockIdx.x + 1, gridDim.x);
    const int ntiles = (row_end - row_begin + pl.TR - 1) / pl.TR;

    /* this thread's slice of the activation vector(s), in registers for the whole phase */
    uint32_t xr[CIT][MT][16];
    float xoff[CIT][MT];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int c = 0; c < CIT; ++c) {
            const int col = ct + c * pl.CT;
            float sx = 0.0f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (active && col < pl.cpr) v = ldg_cg16(xsrc + (size_t)m * pl.K + (size_t)col * 32 + q * 8);
                xr[c][m][4 * q] = v.x; xr[c][m][4 * q + 1] = v.y; xr[c][m][4 * q + 2] = v.z; xr[c][m][4 * q + 3] = v.w;
                sx += bf16_lo(v.x) + bf16_hi(v.x) + bf16_lo(v.y) + bf16_hi(v.y) + bf16_lo(v.z) + bf16_hi(v.z) +
                      bf16_lo(v.w) + bf16_hi(v.w);
            }
            xoff[c][m] = 136.0f * sx;
        }

    /* scales of the rows this thread will touch: one tile ahead, in registers */
    uint16_t sc_next[JTM][PAIRS ? 2 : 1][CIT];
    auto load_scales = [&](int lt) {
        const int rows = min(pl.TR, row_end - (row_begin + lt * pl.TR));
#pragma unroll
        for (int j = 0; j < JTM; ++j) {
            const int p = rg + j * pl.RG;
            const bool on = active && j < pl.JT && p < rows;
            const size_t r0 = (size_t)(row_begin + lt * pl.TR + p);
#pragma unroll
            for (int c = 0; c < CIT; ++c) {
                const int col = ct + c * pl.CT;
                const bool ok = on && col < pl.cpr;
                sc_next[j][0][c] = ok ? __ldg(pl.s + r0 * pl.G + (col >> 2)) : (uint16_t)0;
                if (PAIRS) sc_next[j][PAIRS ? 1 : 0][c] = ok ? __ldg(pl.s + (r0 + pl.up_offset) * pl.G + (col >> 2)) : (uint16_t)0;
            }
        }
    };
    if (ntiles > 0) load_scales(0);

    for (int lt = 0; lt < ntiles; ++lt) {
        const int tile = tile0 + lt;
        const int s = tile % nstages;
        const int rows = min(pl.TR, row_end - (row_begin + lt * pl.TR));
        uint16_t sc[JTM][PAIRS ? 2 : 1][CIT];
#pragma unroll
        for (int j = 0; j < JTM; ++j)
#pragma unroll
            for (int h = 0; h < (PAIRS ? 2 : 1); ++h)
#pragma unroll
                for (int c = 0; c < CIT; ++c) sc[j][h][c] = sc_next[j][h][c];
        if (lt + 1 < ntiles) load_scales(lt + 1);

        if (!mbar_wait(&sm->full[s], (uint32_t)(tile / nstages) & 1u, &sm->abort_flag)) {
            give_up(sm, sync, ST_CONSUMER_FULL);
            return;
        }
        const uint8_t *st = ring + (size_t)s * stage_bytes;
        const int pslot = tile % kPartSlots;
        if (tile >= kPartSlots) { /* the epilogue must have drained this partial slot */
            if (!mbar_wait(&sm->part_empty[pslot], (uint32_t)(tile / kPartSlots - 1) & 1u, &sm->abort_flag)) {
                give_up(sm, sync, ST_PART_EMPTY);
                return;
            }
        }
        float *part = sm->part[pslot];

#pragma unroll
        for (int j = 0; j < JTM; ++j) {
            if (j >= pl.JT) break;
            const int p = rg + j * pl.RG;
            /* whole half-warps share (rg, j): the branch below is uniform within a half-warp */
            if (!active || p >= rows) continue;
            float val[NVROW];
#pragma unroll
            for (int i = 0; i < NVROW; ++i) val[i] = 0.0f;
#pragma unroll
            for (int c = 0; c < CIT; ++c) {
                const int col = ct + c * pl.CT;
                if (col < pl.cpr) {
                    const uint4 w0 = lds16(st + (size_t)p * pl.rb + (size_t)col * 16);
                    float d0[MT];
#pragma unroll
                    for (int m = 0; m < MT; ++m) d0[m] = 0.0f;
                    chunk_dot<MT>(w0, xr[c], d0);
                    const float s0 = bf16_bits_to_f32(sc[j][0][c]);
#pragma unroll
                    for (int m = 0; m < MT; ++m) val[m] = fmaf(s0, d0[m] - xoff[c][m], val[m]);
                    if (PAIRS) {
                        const uint4 w1 = lds16(st + (size_t)(rows + p) * pl.rb + (size_t)col * 16);
                        float d1[MT];
#pragma unroll
                        for (int m = 0; m < MT; ++m) d1[m] = 0.0f;
                        chunk_dot<MT>(w1, xr[c], d1);
                        const float s1 = bf16_bits_to_f32(sc[j][PAIRS ? 1 : 0][c]);
#pragma unroll
                        for (int m = 0; m < MT; ++m) val[MT + m] = fmaf(s1, d1[m] - xoff[c][m], val[MT + m]);
                    }
                }
            }
            const float r = halfwarp_reduce<NVROW>(val, lane, hmask);
            const int l16 = lane & 15;
            if ((l16 % (16 / NVROW)) == 0) {
                const int vi = l16 / (16 / NVROW);
                part[((size_t)p * NVROW + vi) * pl.nhw + (ct >> 4)] = r;
            }
        }
        __syncwarp();
        if (warp_lane0) {
            mbar_arrive(&sm->empty[s]);          /* the weight stage may be refilled */
            mbar_arrive(&sm->part_full[pslot]);  /* this warp's partials are in place */
        }
    }
}

/* ---- epilogue side of one phase ------------------------------------------------------------ */
template <int MT, bool PAIRS>
__device__ __forceinline__ bool epilogue_phase(const FusedParams &P, const PhasePlan &pl, Smem *sm, int tile0, unsigned seq) {
    constexpr int NVROW = (PAIRS ? 2 : 1) * MT;
    const int lane = threadIdx.x & 31;
    const int row_begin = cta_begin(pl.rows_total, blockIdx.x, gridDim.x);
    const int row_end = cta_begin(pl.rows_total, blockIdx.x + 1, gridDim.x);
    const int ntiles = (row_end - row_begin + pl.TR - 1) / pl.TR;
    for (int lt = 0; lt < ntiles; ++lt) {
        const int tile = tile0 + lt;
        const int pslot = tile % kPartSlots;
        const int rows = min(pl.TR, row_end - (row_begin + lt * pl.TR));
        if (!mbar_wait(&sm->part_full[pslot], (uint32_t)(tile / kPartSlots) & 1u, &sm->abort_flag)) {
            give_up(sm, P.sync, ST_PART_FULL);
            return false;
        }
        const float *part = sm->part[pslot];
        for (int i = lane; i < rows * MT; i += 32) {
            const int p = i / MT, m = i % MT;
            const int row = row_begin + lt * pl.TR + p;
            float a = 0.0f, b = 0.0f;
            const float *pa = part + ((size_t)p * NVROW + m) * pl.nhw;
            for (int h = 0; h < pl.nhw; ++h) a += pa[h];
            if (PAIRS) {
                const float *pb = part + ((size_t)p * NVROW + MT + m) * pl.nhw;
                for (int h = 0; h < pl.nhw; ++h) b += pb[h];
                const float g = round_bf16(a), u = round_bf16(b);
                P.act[(size_t)m * P.I + row] = f32_to_bf16_bits(silu_mul(g, u));
            } else if (P.tp == 1) {
                float y = round_bf16(a);
                if (P.residual) {
                    y = round_bf16(bf16_bits_to_f32(P.residual[(size_t)m * P.H + row]) + y);
                    P.residual[(size_t)m * P.H + row] = f32_to_bf16_bits(y);
                }
                P.out[(size_t)m * P.H + row] = f32_to_bf16_bits(y);
            } else {
                const size_t off = (size_t)((seq & 1u) * P.tp + P.rank) * P.slot_stride + (size_t)m * P.H + row;
                for (int r = 0; r < P.tp; ++r) P.peer_slots[r][off] = a; /* own slot on every rank */
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->part_empty[pslot]);
    }
    return true;
}

/* ---- the kernel ----------------------------------------------------------------------------- */
template <int CIT1, int CIT2, int MT>
__global__ void __launch_bounds__(kThreads, 1) ffn_fused_kernel(const FusedParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem *sm = (Smem *)smem_raw;
    uint8_t *ring = smem_raw + ((sizeof(Smem) + 127) / 128) * 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ns = P.nstages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ns; ++s) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], kConsumerWarps); }
        for (int s = 0; s < kPartSlots; ++s) { mbar_init(&sm->part_full[s], kConsumerWarps); mbar_init(&sm->part_empty[s], 1); }
        sm->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int b1 = cta_begin(P.p1.rows_total, blockIdx.x, gridDim.x), e1 = cta_begin(P.p1.rows_total, blockIdx.x + 1, gridDim.x);
    const int b2 = cta_begin(P.p2.rows_total, blockIdx.x, gridDim.x), e2 = cta_begin(P.p2.rows_total, blockIdx.x + 1, gridDim.x);
    const int nt1 = (e1 - b1 + P.p1.TR - 1) / P.p1.TR;
    const int nt2 = (e2 - b2 + P.p2.TR - 1) / P.p2.TR;
    const unsigned my_gen = ld_acquire_gpu(P.sync + 1); /* grid-barrier generation at entry */

    if (warp == 0) {
        /* ---------------- producer ---------------- */
        if (lane == 0) {
            int issued = 0;
            for (int t = 0; t < nt1 + nt2; ++t) {
                const int s = t % ns;
                if (t >= ns && !mbar_wait(&sm->empty[s], (uint32_t)(t / ns - 1) & 1u, &sm->abort_flag)) {
                    give_up(sm, P.sync, ST_PRODUCER_EMPTY);
                    break;
                }
                uint8_t *dst = ring + (size_t)s * P.stage_bytes;
                if (t < nt1) {
                    const int r0 = b1 + t * P.p1.TR, rows = min(P.p1.TR, e1 - r0);
                    const uint32_t bytes = (uint32_t)rows * P.p1.rb;
                    mbar_expect_tx(&sm->full[s], 2 * bytes);
                    bulk_g2s(dst, P.p1.w + (size_t)r0 * P.p1.rb, bytes, &sm->full[s]);
                    bulk_g2s(dst + bytes, P.p1.w + (size_t)(r0 + P.p1.up_offset) * P.p1.rb, bytes, &sm->full[s]);
                } else {
                    const int r0 = b2 + (t - nt1) * P.p2.TR, rows = min(P.p2.TR, e2 - r0);
                    const uint32_t bytes = (uint32_t)rows * P.p2.rb;
                    mbar_expect_tx(&sm->full[s], bytes);
                    bulk_g2s(dst, P.p2.w + (size_t)r0 * P.p2.rb, bytes, &sm->full[s]);
                }
                issued = t + 1;
            }
            /* Never leave with a copy of ours still in flight: wait (bounded) for the most recent
             * fill of every stage.  On the normal path the consumers have long seen them. */
            for (int t = max(0, issued - ns); t < issued; ++t) {
                bool done = false;
                for (uint32_t i = 0; i < kSpinLimit && !done; ++i) done = mbar_try_wait(&sm->full[t % ns], (uint32_t)(t / ns) & 1u);
                if (!done) atomicCAS(P.sync + 3, 0u, (unsigned)ST_DRAIN | ((unsigned)blockIdx.x << 8));
            }
        }
    } else if (warp <= kConsumerWarps) {
        /* ---------------- consumers ---------------- */
        consume_phase<CIT1, MT, true>(P.p1, P.x, sm, ring, P.stage_bytes, ns, 0, P.sync);
        /* grid barrier: the whole activation vector must be in global memory before phase 2 */
        if (threadIdx.x == 32) {
            bool ok = false;
            for (uint32_t i = 0; i < kSpinLimit; ++i) {
                if (ld_acquire_gpu(P.sync + 1) != my_gen) { ok = true; break; }
                if ((i & 255) == 255 && sm->abort_flag) break;
                __nanosleep(20);
            }
            if (!ok) give_up(sm, P.sync, ST_GRID_BARRIER);
        }
        named_bar_sync(1, kConsumerThreads);
        if (!sm->abort_flag)
            consume_phase<CIT2, MT, false>(P.p2, P.act, sm, ring, P.stage_bytes, ns, nt1, P.sync);
    } else {
        /* ---------------- epilogue ---------------- */
        /* read before this CTA arrives at the grid barrier: nobody can have advanced it yet */
        const unsigned seq = P.tp > 1 ? ld_acquire_gpu(P.sync + 2) : 0u;
        bool ok = epilogue_phase<MT, true>(P, P.p1, sm, 0, seq);
        /* arrive at the grid barrier: act rows of this CTA are stored */
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            const unsigned prev = atomicAdd(P.sync + 0, 1u);
            if (prev == gridDim.x - 1) {
                atomicExch(P.sync + 0, 0u);
                __threadfence();
                atomicAdd(P.sync + 1, 1u); /* release everybody */
            }
        }
        if (ok) ok = epilogue_phase<MT, false>(P, P.p2, sm, nt1, seq);
        if (P.tp > 1) {
            /* publish this CTA's rows to every rank, wait for every rank's, add in rank order */
            __threadfence_system();
            __syncwarp();
            if (lane < P.tp) red_release_sys_add(P.peer_flags[lane] + blockIdx.x, 1u);
            const unsigned want = (seq + 1u) * (unsigned)P.tp;
            bool arrived = false;
            if (ok) {
                for (uint32_t i = 0; i < kSpinLimit; ++i) {
                    if ((int)(ld_acquire_sys(P.peer_flags[P.rank] + blockIdx.x) - want) >= 0) { arrived = true; break; }
                    __nanosleep(20);
                }
                if (!arrived) give_up(sm, P.sync, ST_PEER_FLAG);
            }
            if (arrived) {
                const float *mine = P.peer_slots[P.rank] + (size_t)(seq & 1u) * P.tp * P.slot_stride;
                for (int i = lane; i < (e2 - b2) * MT; i += 32) {
                    const int row = b2 + i / MT, m = i % MT;
                    float a = 0.0f;
                    for (int r = 0; r < P.tp; ++r) a += ld_relaxed_sys_f32(mine + (size_t)r * P.slot_stride + (size_t)m * P.H + row);
                    float y = round_bf16(a);
                    if (P.residual) {
                        y = round_bf16(bf16_bits_to_f32(P.residual[(size_t)m * P.H + row]) + y);
                        P.residual[(size_t)m * P.H + row] = f32_to_bf16_bits(y);
                    }
                    P.out[(size_t)m * P.H + row] = f32_to_bf16_bits(y);
                }
            }
        }
    }
    __syncthreads();
    /* the call sequence number advances once per launch (parity of the peer slots, flag target) */
    if (blockIdx.x == 0 && threadIdx.x == 0 && P.tp > 1) atomicAdd(P.sync + 2, 1u);
}


/* ============================================================================================= */
/* Host side: per-device state, the tiling plan, the launch                                      */
/* ============================================================================================= */

struct DeviceState {
    bool ready = false;
    int sm_count = 0;
    int smem_optin = 0;
    int cooperative = 0;
    unsigned *sync = nullptr; /* 4 words: count, generation, sequence, status */
    bool attr_set[2][2][2] = {};
};
static DeviceState g_dev[64];
static std::mutex g_dev_mutex;

static int device_state(DeviceState **out) {
    int dev = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FFN_ERR_CONFIG, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState &d = g_dev[dev];
    if (!d.ready) {
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev), "SM count");
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "smem opt-in");
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.cooperative, cudaDevAttrCooperativeLaunch, dev), "cooperative launch");
        if (cudaMalloc(&d.sync, 4 * sizeof(unsigned)) != cudaSuccess)
            return fail(FFN_ERR_ALLOC, "cannot allocate the kernel's synchronisation words");
        FFN_CUDA_TRY(cudaMemset(d.sync, 0, 4 * sizeof(unsigned)), "clear synchronisation words");
        d.ready = true;
    }
    *out = &d;
    return FFN_OK;
}

static int round_up(int v, int m) { return (v + m - 1) / m * m; }

/* Pick column threads / row groups for one phase.  Returns false when the row does not fit. */
static bool plan_phase(PhasePlan &pl, int K, int MT, bool pairs, int target_bytes, int &cit_out) {
    pl.K = K; pl.rb = K / 2; pl.cpr = K / 32; pl.G = K / FFN_INT4_GROUP;
    double best = -1.0;
    int best_cit = 0;
    for (int cit = 1; cit <= 2; ++cit) {
        if (MT * cit > 2) continue; /* register budget: at most 32 activation registers */
        const int ct = round_up((pl.cpr + cit - 1) / cit, 16);
        if (ct > kConsumerThreads) continue;
        int rg = kConsumerThreads / ct;
        if (pairs) rg = min(rg, max(1, target_bytes / (2 * pl.rb)));
        else rg = min(rg, max(1, (kMaxJT * target_bytes) / pl.rb)); /* never binding in practice */
        double util = (double)pl.cpr / (ct * cit) * (double)(ct * rg) / kConsumerThreads;
        util += 0.02 * cit; /* ties: more work per reduction */
        if (util > best) { best = util; best_cit = cit; }
    }
    if (!best_cit) return false;
    const int cit = best_cit;
    pl.CT = round_up((pl.cpr + cit - 1) / cit, 16);
    pl.RG = kConsumerThreads / pl.CT;
    if (pairs) {
        pl.RG = min(pl.RG, max(1, target_bytes / (2 * pl.rb)));
        pl.JT = 1;
    } else {
        pl.JT = max(1, min(kMaxJT, target_bytes / (pl.RG * pl.rb)));
    }
    pl.TR = pl.JT * pl.RG;
    pl.nhw = pl.CT / 16;
    cit_out = cit;
    return true;
}

template <int C1, int C2, int MT>
static int launch_fused(DeviceState &d, const FusedParams &P, int grid, size_t smem, cudaStream_t stream) {
    bool &set = d.attr_set[C1 - 1][C2 - 1][MT - 1];
    if (!set) {
        FFN_CUDA_TRY(cudaFuncSetAttribute(ffn_fused_kernel<C1, C2, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          d.smem_optin), "fused FFN: shared-memory opt-in");
        set = true;
    }
    void *args[] = {(void *)&P};
    FFN_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)ffn_fused_kernel<C1, C2, MT>, dim3(grid), dim3(kThreads),
                                             args, smem, stream), "fused FFN launch");
    return FFN_OK;
}

int fused_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                     const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual) {
    if (tokens < 1 || tokens > 2) return FFN_NOT_ADMITTED;
    DeviceState *dp = nullptr;
    const int st = device_state(&dp);
    if (st) return st;
    DeviceState &d = *dp;
    if (!d.cooperative) return FFN_NOT_ADMITTED;
    if (((uintptr_t)w->gate_up_i4 & 15) || ((uintptr_t)w->down_i4 & 15) || ((uintptr_t)normed & 15) ||
        ((uintptr_t)act & 15))
        return FFN_NOT_ADMITTED;

    FusedParams P = {};
    P.x = (const uint16_t *)normed;
    P.act = (uint16_t *)act;
    P.out = (uint16_t *)layer_out;
    P.M = tokens; P.H = H; P.I = I;
    P.sync = d.sync;
    P.tp = 1; P.rank = 0;
    P.residual = (uint16_t *)residual;
    if (tp && tp->tp > 1) {
        P.tp = tp->tp; P.rank = tp->rank;
        P.peer_slots = tp->peer_slots; P.peer_flags = tp->peer_flags; P.slot_stride = tp->slot_stride;
        if (tokens * H > tp->slot_stride) return fail(FFN_ERR_CONFIG, "fused FFN: %d tokens exceed the exchange buffer", tokens);
    }
    const int target = 36 * 1024;
    int c1 = 0, c2 = 0;
    if (!plan_phase(P.p1, H, tokens, true, target, c1)) return FFN_NOT_ADMITTED;
    if (!plan_phase(P.p2, I, tokens, false, target, c2)) return FFN_NOT_ADMITTED;
    P.p1.w = w->gate_up_i4; P.p1.s = (const uint16_t *)w->gate_up_i4_scales;
    P.p1.rows_total = I; P.p1.up_offset = I;
    P.p2.w = w->down_i4; P.p2.s = (const uint16_t *)w->down_i4_scales;
    P.p2.rows_total = H; P.p2.up_offset = 0;
    if (P.p1.TR * 2 * tokens * P.p1.nhw > kPartFloats || P.p2.TR * tokens * P.p2.nhw > kPartFloats)
        return FFN_NOT_ADMITTED;
    P.stage_bytes = round_up(max(2 * P.p1.TR * P.p1.rb, P.p2.TR * P.p2.rb), 128);
    const size_t fixed = ((sizeof(Smem) + 127) / 128) * 128;
    P.nstages = (int)min((size_t)kMaxStages, ((size_t)d.smem_optin - fixed) / (size_t)P.stage_bytes);
    if (P.nstages < 2) return FFN_NOT_ADMITTED;
    const size_t smem = fixed + (size_t)P.nstages * P.stage_bytes;
    int grid = d.sm_count;
    if (tp && tp->tp > 1) {
        grid = min(grid, tp->max_ctas); /* every rank must use the same grid: CTA c pairs with CTA c */
    }

#define FFN_LAUNCH(A, B, C) return launch_fused<A, B, C>(d, P, grid, smem, stream)
    if (tokens == 1) {
        if (c1 == 1 && c2 == 1) FFN_LAUNCH(1, 1, 1);
        if (c1 == 1 && c2 == 2) FFN_LAUNCH(1, 2, 1);
        if (c1 == 2 && c2 == 1) FFN_LAUNCH(2, 1, 1);
        FFN_LAUNCH(2, 2, 1);
    }
    FFN_LAUNCH(1, 1, 2);
#undef FFN_LAUNCH
}

int fused_ffn_try(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                  const FfnMlpWeights *w, int tokens, int H, int I) {
    return fused_ffn_launch(stream, normed, act, layer_out, w, tokens, H, I, nullptr, nullptr);
}

int fused_status(unsigned *status_out, bool reset) {
    DeviceState *dp = nullptr;
    const int st = device_state(&dp);
    if (st) return st;
    unsigned words[4];
    FFN_CUDA_TRY(cudaMemcpy(words, dp->sync, sizeof(words), cudaMemcpyDeviceToHost), "read kernel status");
    *status_out = words[3];
    if (reset && words[3] != 0) FFN_CUDA_TRY(cudaMemset(dp->sync, 0, sizeof(words)), "reset synchronisation words");
    return FFN_OK;
}

int gemm_int4_dispatch(const void *a, const void *packed, const void *scales, void *out, int M, int N,
                       int K, cudaStream_t stream) {
    return gemm_int4_generic(a, packed, scales, out, nullptr, M, N, K, stream);
}

}  // namespace ffn
