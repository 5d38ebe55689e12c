/*
 * stream_common.cuh - device helpers shared by the streaming decode kernels (ffn_fused.cu: the
 * row-major single-launch kernel; ffn_kmajor.cu: the kernel over the k-major copy of the down
 * projection): role geometry, mbarrier / bulk-copy wrappers with bounded waits, the block-fixed-point
 * form of an activation slice, the dp4a inner product over widened INT4 codes, the transposed
 * half-warp reduction.
 */
#pragma once

#include "common.cuh"

namespace ffn {

constexpr int kConsumerWarps = 17;
constexpr int kConsumerThreads = kConsumerWarps * 32;  /* 544 = 17 * 32: I = 17408 = 17 * 1024 */
constexpr int kThreads = (kConsumerWarps + 2) * 32;    /* 608 */
constexpr int kMaxStages = 8;
constexpr int kPartSlots = 4;
constexpr int kPartFloats1 = 160;                      /* floats per partial slot, one token: JT*NVROW*RG*CT/16 <= 4*544/16 = 136 */
constexpr int kPartFloats2 = 288;                      /* two tokens: <= 8*544/16 = 272 */
constexpr int kMaxJT = 4;                              /* row steps per thread per tile */
constexpr uint32_t kSpinLimit = 1u << 22;              /* bounded waits: polls of >= 32..100 ns, i.e. 0.15 .. 0.5 s */

/* status word values (where a wait gave up) */
enum { ST_OK = 0, ST_PRODUCER_EMPTY = 1, ST_CONSUMER_FULL = 2, ST_PART_EMPTY = 3, ST_PART_FULL = 4,
       ST_GRID_BARRIER = 5, ST_PEER_DATA = 6, ST_DRAIN = 7, ST_X_FULL = 8,
       ST_PARTIALS = 9 /* the other CTAs' partial sums */, ST_NEXT_X = 10 /* the residual stream of the next layer */,
       ST_ACT_READY = 11 /* this CTA's own activations */ };

struct PhasePlan {
    const uint8_t *w;     /* packed rows */
    const uint16_t *s;    /* scales */
    int K, rb, cpr, G;    /* columns, row bytes, 16-byte chunks per row, groups per row */
    int CT, RG, JT, TR;   /* column threads, row groups, row steps per tile, rows(pairs) per tile */
    int rows_total;       /* rows (phase 2) or gate/up pairs (phase 1) this rank owns */
    int up_offset;        /* phase 1: row index of up row 0 (= local I) */
    int nhw;              /* half-warps per row group = CT / 16 */
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
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) { /* never suspends */
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
/* Bounded wait.  Returns false when the limit ran out or another thread already gave up.  A
 * waiting warp sleeps between polls so that it does not take issue slots from the arithmetic
 * warps: SLEEP_NS is short for the consumers (they wait for data) and longer for the producer and
 * the epilogue, which wait most of the time. */
template <int SLEEP_NS>
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        __nanosleep(SLEEP_NS);
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255) == 255 && *abort_flag) return false;
    }
    return false;
}
/* Programmatic dependent launch.  griddep_launch lets the next grid of the stream be scheduled onto
 * SMs as this grid's CTAs leave them; griddep_wait returns once every grid this launch depends on has
 * completed and its writes are visible.  Both do nothing in a launch without the attribute. */
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint4 lds16_at(uint32_t addr) { /* addr: shared-window byte address */
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_bf16_at(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __uint_as_float((uint32_t)v << 16);
}
__device__ __forceinline__ uint4 lds16(const void *p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); /* (a & b) ^ c */
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { /* signed bytes x signed bytes */
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) { /* signed bytes x unsigned bytes */
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

/* ---- activations as block fixed point ------------------------------------------------------- */
/* One thread's 32-element slice of an activation vector, prepared once per phase:
 *   X_k = rint(x_k * 2^(14-E)),  E = exponent of the largest |x_k| of the slice, so |X_k| < 2^15.
 * A BF16 value has 8 significant bits, so every element within 2^-7 of the slice maximum is held
 * exactly; smaller ones lose only bits below max*2^-15.  X is stored as byte planes laid out for
 * dp4a against the widened weight bytes: word j (codes k = 8j..8j+7) pairs
 *   even codes k = 8j + {0,2,4,6}  with  he[j] (high bytes, signed) and le[j] (low bytes, unsigned)
 *   odd  codes k = 8j + {1,3,5,7}  with  ho[j] / lo[j].
 * fac = 2^(E-14) / 16 undoes the scaling of X and the factor 16 the widened codes carry. */
struct XChunk {
    uint32_t he[4], ho[4], le[4], lo[4];
    float fac;
};

/* The 32 BF16 values of one slice (64-byte aligned): from global memory (x, present when the kernel
 * starts) or from the shared-memory copy of act the producer fetched. */
template <bool GLOBAL>
__device__ __forceinline__ void load_chunk(uint32_t (&v)[16], const uint16_t *src, bool on) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint4 t = make_uint4(0, 0, 0, 0);
        if (on) t = GLOBAL ? __ldg((const uint4 *)(src + q * 8)) : lds16(src + q * 8);
        v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
}

__device__ __forceinline__ void prepare_chunk(XChunk &xc, uint32_t (&v)[16], bool on,
                                              const uint16_t *norm_w = nullptr /* global, this chunk's 32 weights */,
                                              float inv_rms = 1.0f, float gemma = 0.0f) {
    if (norm_w != nullptr && on) { /* fused RMSNorm: the reference's expression and its BF16 rounding */
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 wq = __ldg((const uint4 *)(norm_w + q * 8));
            const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float lo = bf16_lo(v[4 * q + i]) * inv_rms * (bf16_lo(ww[i]) + gemma);
                const float hi = bf16_hi(v[4 * q + i]) * inv_rms * (bf16_hi(ww[i]) + gemma);
                v[4 * q + i] = (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
            }
        }
    }
    uint32_t mx = 0; /* per-halfword maximum of the magnitude bits */
#pragma unroll
    for (int i = 0; i < 16; ++i) mx = __vmaxu2(mx, v[i] & 0x7FFF7FFFu);
    const uint32_t top = max(mx & 0xFFFFu, mx >> 16);
    const int E = (int)(top >> 7); /* biased exponent of the largest magnitude */
    /* E < 19 (|x| < 2^-108) is treated as an all-zero slice.  A slice that holds an Inf or a NaN
     * (E == 255) gets fac = NaN, so every row's sum becomes NaN: non-finite inputs give non-finite
     * outputs, as the reference's FMA chain does (csrc/kernels/gemm_quant.cu:182-199), at no cost
     * in the inner loop. */
    const bool live = E >= 19 && E < 255;
    const float up = live ? __uint_as_float((uint32_t)(268 - E) << 23) : 0.0f;   /* 2^(141-E) */
    xc.fac = live ? __uint_as_float((uint32_t)(E - 18) << 23)                    /* 2^(E-141) / 16 */
                  : (E == 255 ? __uint_as_float(0x7FC00000u) : 0.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int X[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            /* 1.5*2^23 + x*up has the rounded (nearest-even) integer in its low mantissa bits; only
             * the low 16 bits are used below and 0x4B400000 contributes none of them */
            X[2 * i] = __float_as_int(fmaf(bf16_lo(v[4 * j + i]), up, 12582912.0f));
            X[2 * i + 1] = __float_as_int(fmaf(bf16_hi(v[4 * j + i]), up, 12582912.0f));
        }
        /* bytes 0/1 of each X are its low/high byte (two's complement 16-bit) */
        const uint32_t e02 = prmt(X[0], X[2], 0x5140), e46 = prmt(X[4], X[6], 0x5140); /* lo0 lo2 hi0 hi2 */
        const uint32_t o13 = prmt(X[1], X[3], 0x5140), o57 = prmt(X[5], X[7], 0x5140);
        xc.le[j] = prmt(e02, e46, 0x5410);
        xc.he[j] = prmt(e02, e46, 0x7632);
        xc.lo[j] = prmt(o13, o57, 0x5410);
        xc.ho[j] = prmt(o13, o57, 0x7632);
    }
}

/* 16 * sum_k code_k * X_k over one 16-byte chunk.  A 4-bit two's-complement code placed in the high
 * nibble of a byte IS the signed byte 16*code, so (w & 0xF0F0F0F0) holds the odd codes of a word
 * and ((w << 4) & 0xF0F0F0F0) the even ones, ready for a signed dp4a: one shift and two ANDs widen
 * eight codes, with no offset to remove afterwards.  Integer arithmetic, exact (|sum| < 2^27). */
__device__ __forceinline__ int chunk_dot(const uint4 &w, const XChunk &xc) {
    int hi = 0, lo = 0;
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t o = ws[j] & 0xF0F0F0F0u;
        const uint32_t e = (ws[j] << 4) & 0xF0F0F0F0u;
        hi = dp4a_ss(e, xc.he[j], hi);
        hi = dp4a_ss(o, xc.ho[j], hi);
        lo = dp4a_su(e, xc.le[j], lo);
        lo = dp4a_su(o, xc.lo[j], lo);
    }
    return hi * 256 + lo;
}

/* Sum of NV values over the 16 lanes of a half-warp; value i ends up in lane (16/NV)*i of the
 * half-warp.  NV in {1, 2, 4}. */
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

/* ---- host-side tiling helpers --------------------------------------------------------------- */
constexpr int kDefaultStageTarget = 62 * 1024; /* bytes of weights per stage the planner aims for */
static inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

/* Pick column threads / row groups for one phase.  Returns false when the row does not fit. */
static inline bool plan_phase(PhasePlan &pl, int K, int MT, bool pairs, int target_bytes, int &cit_out) {
    pl.K = K; pl.rb = K / 2; pl.cpr = K / 32; pl.G = K / FFN_INT4_GROUP;
    double best = -1.0;
    int best_cit = 0;
    for (int cit = 1; cit <= 2; ++cit) {
        if (MT * cit > 2) continue; /* register budget: at most two prepared activation chunks */
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
        pl.JT = max(1, min(2, target_bytes / (2 * pl.RG * pl.rb)));
    } else {
        pl.JT = max(1, min(kMaxJT, target_bytes / (pl.RG * pl.rb)));
    }
    pl.TR = pl.JT * pl.RG;
    pl.nhw = pl.CT / 16;
    cit_out = cit;
    return true;
}

}  // namespace ffn
