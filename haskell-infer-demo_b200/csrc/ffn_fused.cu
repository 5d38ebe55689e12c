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
 *                 in flight while the grid waits for the activation vector.  It also brings the
 *                 activation vector of each phase into shared memory (x at entry, act as soon as
 *                 the grid barrier opens).
 *   warps 1..17   consumers: thread (ct, rg) owns 16-byte column chunk(s) ct of every row r with
 *                 r % RG == rg of a tile.  Its 32-element slice of the activation vector lives in
 *                 registers for the whole phase, as 16-bit block-fixed-point split into byte planes;
 *                 the 4-bit codes are widened to bytes with one logic op per four codes and
 *                 multiplied with dp4a (exact integer arithmetic inside a 32-code chunk), then
 *                 scaled once per chunk in FP32.  Half-warp shuffles reduce the row partials.
 *   warp 18       epilogue: adds the half-warp partials in a fixed order (deterministic), applies
 *                 the reference's rounding points, stores act / y, runs the grid barrier arrival and
 *                 the cross-GPU exchange.
 *
 * Cross-rank reduce (TP = R > 1): CTA c of every rank owns the same output rows.  Its epilogue
 * sends the FP32 partial sums of those rows into slot `rank` of a [2][R][M][H] buffer in EVERY rank's
 * memory (peer stores over NVLink), each as one 8-byte word {value, call number + 1}, tile by tile
 * while phase 2 runs; at the end it polls (bounded) the words of its own rows in its own memory
 * until all R carry this call's number, adds them in rank order and rounds once to BF16.  No fence,
 * no flag, no collective call and no second kernel.
 *
 * Every device-side wait is bounded; on expiry the kernel records where it gave up in the status
 * word, drains its own copies and returns.  The host maps that to FFN_ERR_CUDA.
 */
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "stream_common.cuh"

namespace ffn {

struct FusedParams {
    const uint16_t *x;    /* [M][H] bf16 */
    uint16_t *act;        /* [M][I] bf16 (global scratch the caller's workspace provides) */
    uint16_t *out;        /* [M][H] bf16 */
    PhasePlan p1, p2;
    int M, H, I;
    int stage_bytes, nstages, xs_bytes;
    int stage_w_bytes;    /* weights part of a stage; the tile's scales follow it */
    int sc_half_bytes;    /* room for one contiguous run of scales (gate or up) incl. 16 bytes of slack */
    unsigned *sync;       /* [0] arrivals (monotonic), [1] arrivals at the end of the previous launch,
                             [2] unused, [3] status */
    /* tensor parallelism (tp == 1: unused) */
    int tp, rank;
    unsigned long long *const *peer_slots; /* device array [tp]: each rank's [2][tp][M_max][H] tagged words */
    int slot_stride;      /* elements per (parity, rank) slot = M_max * H */
    unsigned *tp_seq;     /* this communicator's call counter (slot parity, tag of the exchanged words) */
    /* optional fused residual update with the reduced output y: h <- bf16(h + y); NULL = off */
    uint16_t *residual;
    /* optional fused RMSNorm of the input (x is then the residual stream h): n = bf16(h * rsqrt(mean(h^2)
     * + eps) * (w + gemma)); NULL = x is already normalized */
    const uint16_t *norm_w;
    float norm_eps;
    int norm_gemma;
    long long *trace;     /* optional [CTAs][16] global-timer stamps of every CTA's pipeline events (NULL = off) */
    int early_weights;    /* 1: the first fill of every stage is issued before the wait on the previous launch of
                             the stream (set by the host together with the dependent-launch attribute) */
    int gemv;             /* 1: single-matrix mode - only phase 2 runs, its activation is the caller's input
                             (no grid barrier, nothing handed over between phases) */
#ifdef FFN_INT4_TUNING
    int debug;            /* measurement build only: bit 0 skips the arithmetic, bit 1 skips the weight copies */
#endif
};
#ifdef FFN_INT4_TUNING
#define FFN_DEBUG_BIT(P, b) ((P).debug & (b))
#else
#define FFN_DEBUG_BIT(P, b) 0
#endif

struct Smem;
__host__ __device__ constexpr size_t fused_smem_header(int tokens); /* bytes before the activation copy */
struct Smem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t part_full[kPartSlots];
    uint64_t part_empty[kPartSlots];
    uint64_t x_full[2];
    int abort_flag;
    int pad[11];
    float norm_red[2][kConsumerWarps + 3];
    float part[1]; /* kPartSlots slots of kPartFloats1 or kPartFloats2 floats follow (sized by the token count) */
};

__host__ __device__ constexpr size_t fused_smem_header(int tokens) {
    return (sizeof(Smem) + (size_t)kPartSlots * (tokens == 1 ? kPartFloats1 : kPartFloats2) * sizeof(float) + 127) / 128 * 128;
}

__device__ __forceinline__ void give_up(Smem *sm, unsigned *sync, int where) {
    sm->abort_flag = 1;
    atomicCAS(sync + 3, 0u, (unsigned)where | ((unsigned)blockIdx.x << 8));
}

/* first row of CTA `cta`'s contiguous share; total * ctas < 2^32 is checked on the host */
__device__ __forceinline__ int cta_begin(int total, int cta, int ctas) {
    return (int)(((unsigned)total * (unsigned)cta) / (unsigned)ctas);
}

__device__ __forceinline__ void stamp(const FusedParams &P, int slot) {
    if (P.trace) { /* every CTA, global timer: [cta][16] */
        long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        P.trace[blockIdx.x * 16 + slot] = t;
    }
}

/* ---- consumer side of one phase ------------------------------------------------------------ */
template <int CIT, int MT, bool PAIRS>
__device__ __forceinline__ void consume_phase(const FusedParams &P, const PhasePlan &pl, Smem *sm,
                                              const uint16_t *xs, uint8_t *ring, int tile0) {
    constexpr int NVROW = (PAIRS ? 2 : 1) * MT;
    constexpr int VALS = 4 * MT;   /* values a thread carries through a tile: one transposed reduction per four */
    constexpr int JTM = VALS / NVROW; /* row steps per thread per tile: 2 of pairs, 4 of single rows */
    const int stage_bytes = P.stage_bytes, nstages = P.nstages;
    const uint32_t ring_addr = smem_u32(ring);
    const int ti = threadIdx.x - 32;
    const int lane = threadIdx.x & 31;
    const bool active = ti < pl.CT * pl.RG;
    const int ct = ti % pl.CT, rg = ti / pl.CT;
    const unsigned hmask = 0xFFFFu << (lane & 16);
    const int row_begin = cta_begin(pl.rows_total, blockIdx.x, gridDim.x);
    const int row_end = cta_begin(pl.rows_total, blockIdx.x + 1, gridDim.x);
    const int ntiles = (row_end - row_begin + pl.TR - 1) / pl.TR;

    /* This thread's 32-element slice(s) of the activation vector(s).  Phase 1 reads x straight from
     * global memory: it is there when the kernel starts, so the loads are in flight while the
     * producer is still setting up.  Phase 2 waits for the copy of act the producer brings into
     * shared memory once the grid barrier has opened. */
    const bool direct = PAIRS || P.gemv; /* single-matrix mode: the activation is an input too */
    if (!direct && !mbar_wait<64>(&sm->x_full[1], 0u, &sm->abort_flag)) {
        give_up(sm, P.sync, ST_X_FULL);
        return;
    }
    const uint16_t *src = direct ? P.x : xs;
    uint32_t xv[CIT][MT][16];
#pragma unroll
    for (int c = 0; c < CIT; ++c)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int col = ct + c * pl.CT;
            const uint16_t *from = src + (size_t)m * pl.K + (size_t)min(col, pl.cpr - 1) * 32;
            if (direct) load_chunk<true>(xv[c][m], from, active && col < pl.cpr);
            else load_chunk<false>(xv[c][m], from, active && col < pl.cpr);
        }
    float inv_rms[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) inv_rms[m] = 1.0f;
    const bool normalize = PAIRS && P.norm_w != nullptr;
    if (normalize) { /* every CTA needs the whole normalized vector, so every CTA takes the (cheap) norm */
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float ss = 0.0f;
            if (rg == 0) { /* row group 0 covers every slice exactly once; absent slices hold zeros */
#pragma unroll
                for (int c = 0; c < CIT; ++c)
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t pr = xv[c][m][i];
                        ss = fmaf(bf16_lo(pr), bf16_lo(pr), ss);
                        ss = fmaf(bf16_hi(pr), bf16_hi(pr), ss);
                    }
            }
            ss = warp_sum(ss);
            if (lane == 0) sm->norm_red[m][ti >> 5] = ss;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) total += sm->norm_red[m][w];
            inv_rms[m] = rsqrtf(total / (float)pl.K + P.norm_eps);
        }
    }
    XChunk xc[CIT][MT];
#pragma unroll
    for (int c = 0; c < CIT; ++c)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int col = ct + c * pl.CT;
            const bool on = active && col < pl.cpr;
            prepare_chunk(xc[c][m], xv[c][m], on,
                          normalize ? P.norm_w + (size_t)min(col, pl.cpr - 1) * 32 : nullptr, inv_rms[m],
                          P.norm_gemma ? 1.0f : 0.0f);
        }
    if (threadIdx.x == 32) stamp(P, PAIRS ? 2 : 7);

    for (int lt = 0; lt < ntiles; ++lt) {
        const int tile = tile0 + lt;
        const int s = tile % nstages;
        const int rows = min(pl.TR, row_end - (row_begin + lt * pl.TR));
        if (!mbar_wait<32>(&sm->full[s], (uint32_t)(tile / nstages) & 1u, &sm->abort_flag)) {
            give_up(sm, P.sync, ST_CONSUMER_FULL);
            return;
        }
        if (threadIdx.x == 32 && lt == 0) stamp(P, PAIRS ? 3 : 8);
        /* 32-bit shared-window addresses from here on.  The tile's scales sit behind its weights;
         * a run starts where the global run does modulo 16 (the copy was widened down to a 16-byte
         * boundary). */
        const int row0 = row_begin + lt * pl.TR;
        const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)stage_bytes;
        const uint32_t sc0 = st + (uint32_t)P.stage_w_bytes + (((uint32_t)row0 * (uint32_t)pl.G * 2u) & 15u);
        const uint32_t sc1 = st + (uint32_t)(P.stage_w_bytes + P.sc_half_bytes) +
                             (((uint32_t)(row0 + pl.up_offset) * (uint32_t)pl.G * 2u) & 15u);
        const int pslot = tile % kPartSlots;
        if (tile >= kPartSlots) { /* the epilogue must have drained this partial slot */
            if (!mbar_wait<100>(&sm->part_empty[pslot], (uint32_t)(tile / kPartSlots - 1) & 1u, &sm->abort_flag)) {
                give_up(sm, P.sync, ST_PART_EMPTY);
                return;
            }
        }
        float *part = sm->part + (size_t)pslot * (MT == 1 ? kPartFloats1 : kPartFloats2);

        /* all row steps of the tile first, then ONE transposed half-warp reduction of up to four
         * values (row step x gate/up x token) instead of one reduction per row */
        float val[VALS];
#pragma unroll
        for (int v = 0; v < VALS; ++v) val[v] = 0.0f;
        if (active && !FFN_DEBUG_BIT(P, 1)) {
            /* No data-dependent branches in here: a column chunk past the row end reads a clamped
             * address against an all-zero prepared slice, a row past the tile end reads the tile's
             * last row and its value is dropped at the store.  That leaves the compiler free to
             * overlap the shared-memory loads and the integer chains of all chunks of a row step. */
            const uint32_t up_bytes = (uint32_t)rows * (uint32_t)pl.rb;
            uint32_t coff[CIT], soff[CIT];
#pragma unroll
            for (int c = 0; c < CIT; ++c) {
                const int col = min(ct + c * pl.CT, pl.cpr - 1);
                coff[c] = (uint32_t)col * 16u;
                soff[c] = (uint32_t)(col >> 2) * 2u;
            }
#pragma unroll
            for (int j = 0; j < JTM; ++j) {
                if (j < pl.JT) { /* uniform over the CTA */
                    const int pj = min(rg + j * pl.RG, rows - 1);
                    const uint32_t wp = st + (uint32_t)pj * (uint32_t)pl.rb;
                    const uint32_t s0p = sc0 + (uint32_t)pj * (uint32_t)pl.G * 2u, s1p = sc1 + (uint32_t)pj * (uint32_t)pl.G * 2u;
                    uint4 w0[CIT], w1[CIT];
                    float f0[CIT], f1[CIT];
#pragma unroll
                    for (int c = 0; c < CIT; ++c) {
                        w0[c] = lds16_at(wp + coff[c]);
                        f0[c] = lds_bf16_at(s0p + soff[c]);
                        if (PAIRS) {
                            w1[c] = lds16_at(wp + up_bytes + coff[c]);
                            f1[c] = lds_bf16_at(s1p + soff[c]);
                        }
                    }
#pragma unroll
                    for (int c = 0; c < CIT; ++c) {
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            val[j * NVROW + m] = fmaf((float)chunk_dot(w0[c], xc[c][m]), f0[c] * xc[c][m].fac, val[j * NVROW + m]);
                            if (PAIRS)
                                val[j * NVROW + MT + m] = fmaf((float)chunk_dot(w1[c], xc[c][m]), f1[c] * xc[c][m].fac, val[j * NVROW + MT + m]);
                        }
                    }
                }
            }
            /* whole half-warps are active or not (CT is a multiple of 16) */
            const int l16 = lane & 15;
#pragma unroll
            for (int q = 0; q < VALS / 4; ++q) {
                float four[4] = {val[4 * q], val[4 * q + 1], val[4 * q + 2], val[4 * q + 3]};
                const float r = halfwarp_reduce<4>(four, lane, hmask);
                if ((l16 & 3) == 0) {
                    const int v = 4 * q + (l16 >> 2), j = v / NVROW, i = v % NVROW, p = rg + j * pl.RG;
                    if (j < pl.JT && p < rows) part[((size_t)p * NVROW + i) * pl.nhw + (ct >> 4)] = r;
                }
            }
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(&sm->empty[s]);          /* the weight stage may be refilled */
            mbar_arrive(&sm->part_full[pslot]);  /* this warp's partials are in place */
        }
    }
    if (threadIdx.x == 32) stamp(P, PAIRS ? 4 : 9);
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
        if (!mbar_wait<100>(&sm->part_full[pslot], (uint32_t)(tile / kPartSlots) & 1u, &sm->abort_flag)) {
            give_up(sm, P.sync, ST_PART_FULL);
            return false;
        }
        const float *part = sm->part + (size_t)pslot * (MT == 1 ? kPartFloats1 : kPartFloats2);
        for (int i = lane; i < rows * MT; i += 32) {
            const int p = i / MT, m = i % MT;
            const int row = row_begin + lt * pl.TR + p;
            float a = 0.0f, b = 0.0f;
            const float *pa = part + ((size_t)p * NVROW + m) * pl.nhw;
#pragma unroll 4
            for (int h = 0; h < pl.nhw; ++h) a += pa[h];
            if (PAIRS) {
                const float *pb = part + ((size_t)p * NVROW + MT + m) * pl.nhw;
#pragma unroll 4
                for (int h = 0; h < pl.nhw; ++h) b += pb[h];
                const float g = round_bf16(a), u = round_bf16(b);
                P.act[(size_t)m * P.I + row] = f32_to_bf16_bits(silu_mul(g, u));
            } else if (P.tp == 1) {
                const float y = round_bf16(a);
                P.out[(size_t)m * P.H + row] = f32_to_bf16_bits(y);
                if (P.residual)
                    P.residual[(size_t)m * P.H + row] =
                        f32_to_bf16_bits(bf16_bits_to_f32(P.residual[(size_t)m * P.H + row]) + y);
            } else {
                const size_t off = (size_t)((seq & 1u) * P.tp + P.rank) * P.slot_stride + (size_t)m * P.H + row;
                for (int r = 0; r < P.tp; ++r) tp_store_tagged(P.peer_slots[r] + off, a, tp_tag(seq)); /* own slot on every rank */
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
    uint16_t *xs = (uint16_t *)(smem_raw + fused_smem_header(MT));
    uint8_t *ring = (uint8_t *)xs + P.xs_bytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ns = P.nstages;

    if (threadIdx.x == 0) griddep_launch(); /* the next launch may take this CTA's SM the moment it is free */
    if (warp == 0) {
        if (lane == 0) stamp(P, 0);
        if (lane < ns) { mbar_init(&sm->full[lane], 1); mbar_init(&sm->empty[lane], kConsumerWarps); }
        if (lane >= 8 && lane < 8 + kPartSlots) { mbar_init(&sm->part_full[lane - 8], kConsumerWarps); mbar_init(&sm->part_empty[lane - 8], 1); }
        if (lane >= 16 && lane < 18) mbar_init(&sm->x_full[lane - 16], 1);
        if (lane == 31) sm->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int b1 = cta_begin(P.p1.rows_total, blockIdx.x, gridDim.x), e1 = cta_begin(P.p1.rows_total, blockIdx.x + 1, gridDim.x);
    const int b2 = cta_begin(P.p2.rows_total, blockIdx.x, gridDim.x), e2 = cta_begin(P.p2.rows_total, blockIdx.x + 1, gridDim.x);
    const int nt1 = (e1 - b1 + P.p1.TR - 1) / P.p1.TR;
    const int nt2 = (e2 - b2 + P.p2.TR - 1) / P.p2.TR;

    if (warp == 0) {
        /* ---------------- producer ---------------- */
        if (lane == 0) {
            const int total = nt1 + nt2;
            int t = 0;
            auto issue_tile = [&](int t) {
                const int s = t % ns;
                uint8_t *dst = ring + (size_t)s * P.stage_bytes;
                if (FFN_DEBUG_BIT(P, 2)) { mbar_arrive(&sm->full[s]); return; }
                if (t < nt1) {
                    const int r0 = b1 + t * P.p1.TR, rows = min(P.p1.TR, e1 - r0);
                    const uint32_t bytes = (uint32_t)rows * P.p1.rb;
                    /* scale runs widened to 16-byte boundaries (the array's end is one: row counts
                     * are multiples of 8, so N*G*2 is a multiple of 16) */
                    const size_t g0 = (size_t)r0 * P.p1.G * 2, g1 = (size_t)(r0 + P.p1.up_offset) * P.p1.G * 2;
                    const size_t len = (size_t)rows * P.p1.G * 2;
                    const size_t a0 = g0 & ~(size_t)15, a1 = g1 & ~(size_t)15;
                    const uint32_t n0 = (uint32_t)(((g0 + len + 15) & ~(size_t)15) - a0);
                    const uint32_t n1 = (uint32_t)(((g1 + len + 15) & ~(size_t)15) - a1);
                    mbar_expect_tx(&sm->full[s], 2 * bytes + n0 + n1);
                    bulk_g2s(dst, P.p1.w + (size_t)r0 * P.p1.rb, bytes, &sm->full[s]);
                    bulk_g2s(dst + bytes, P.p1.w + (size_t)(r0 + P.p1.up_offset) * P.p1.rb, bytes, &sm->full[s]);
                    bulk_g2s(dst + P.stage_w_bytes, (const uint8_t *)P.p1.s + a0, n0, &sm->full[s]);
                    bulk_g2s(dst + P.stage_w_bytes + P.sc_half_bytes, (const uint8_t *)P.p1.s + a1, n1, &sm->full[s]);
                } else {
                    const int r0 = b2 + (t - nt1) * P.p2.TR, rows = min(P.p2.TR, e2 - r0);
                    const uint32_t bytes = (uint32_t)rows * P.p2.rb;
                    const size_t g0 = (size_t)r0 * P.p2.G * 2, len = (size_t)rows * P.p2.G * 2;
                    const size_t a0 = g0 & ~(size_t)15;
                    const uint32_t n0 = (uint32_t)(((g0 + len + 15) & ~(size_t)15) - a0);
                    mbar_expect_tx(&sm->full[s], bytes + n0);
                    bulk_g2s(dst, P.p2.w + (size_t)r0 * P.p2.rb, bytes, &sm->full[s]);
                    bulk_g2s(dst + P.stage_w_bytes, (const uint8_t *)P.p2.s + a0, n0, &sm->full[s]);
                }
            };
            /* The weights never change, so the first fill of every stage need not wait for the launch
             * before this one in the stream: with programmatic dependent launch this CTA starts as soon
             * as its SM is free, and these copies are in flight while the previous grid drains. */
            if (P.early_weights)
                for (; t < min(ns, total); ++t) issue_tile(t);
            griddep_wait();
            /* grid barrier: every CTA adds one to a monotonic counter; the launch's target is the
             * count the previous launch left behind plus this grid's size (stable during the launch,
             * so replaying a captured graph or changing the grid size needs no host bookkeeping) */
            const unsigned bar_target = P.sync[1] + gridDim.x;
            stamp(P, 1);
            bool act_issued = false, failed = false;
            /* Phase 2's activation vector is fetched once the grid barrier has opened (every CTA has
             * stored its rows of act). */
            auto fetch_act = [&]() {
                bool open = false;
                for (uint32_t i = 0; i < kSpinLimit && !open; ++i) {
                    open = (int)(ld_acquire_gpu(P.sync + 0) - bar_target) >= 0;
                    if (!open) {
                        if ((i & 63) == 63 && sm->abort_flag) break;
                        __nanosleep(32);
                    }
                }
                if (!open) { give_up(sm, P.sync, ST_GRID_BARRIER); failed = true; return; }
                stamp(P, 6);
                mbar_expect_tx(&sm->x_full[1], (uint32_t)(P.M * P.I * 2));
                bulk_g2s(xs, P.act, (uint32_t)(P.M * P.I * 2), &sm->x_full[1]);
                act_issued = true;
            };
            for (; t < total && !failed; ++t) {
                const int s = t % ns;
                /* A stage that still holds a phase-2 tile is only released after the consumers got
                 * the activation vector, so that is the moment to go and wait for the barrier; a
                 * stage holding a phase-1 tile frees up on its own. */
                if (!act_issued && !P.gemv && t - ns >= nt1) { fetch_act(); if (failed) break; }
                if (t >= ns && !mbar_wait<100>(&sm->empty[s], (uint32_t)(t / ns - 1) & 1u, &sm->abort_flag)) {
                    give_up(sm, P.sync, ST_PRODUCER_EMPTY);
                    failed = true;
                    break;
                }
                issue_tile(t);
            }
            if (!act_issued && !failed && !P.gemv) fetch_act();
            /* Never leave with a copy of ours still in flight: wait (bounded) for the most recent
             * fill of every stage and for the activation copies. */
            for (int u = max(0, t - ns); u < t; ++u) {
                bool done = false;
                for (uint32_t i = 0; i < kSpinLimit && !done; ++i) done = mbar_try_wait(&sm->full[u % ns], (uint32_t)(u / ns) & 1u);
                if (!done) atomicCAS(P.sync + 3, 0u, (unsigned)ST_DRAIN | ((unsigned)blockIdx.x << 8));
            }
            if (act_issued) {
                bool done = false;
                for (uint32_t i = 0; i < kSpinLimit && !done; ++i) done = mbar_try_wait(&sm->x_full[1], 0u);
                if (!done) atomicCAS(P.sync + 3, 0u, (unsigned)ST_DRAIN | ((unsigned)blockIdx.x << 8));
            }
        }
    } else if (warp <= kConsumerWarps) {
        /* ---------------- consumers ---------------- */
        griddep_wait(); /* the input may be the previous kernel's output */
        if (!P.gemv) consume_phase<CIT1, MT, true>(P, P.p1, sm, xs, ring, 0);
        if (!sm->abort_flag) consume_phase<CIT2, MT, false>(P, P.p2, sm, xs, ring, nt1);
    } else {
        /* ---------------- epilogue ---------------- */
        griddep_wait(); /* act, out, the residual and the exchange slots may still be in use by the previous launch */
        /* read before this CTA arrives at the grid barrier: nobody can have advanced it yet */
        const unsigned seq = P.tp > 1 ? ld_acquire_gpu(P.tp_seq) : 0u;
        bool ok = true;
        if (!P.gemv) {
            ok = epilogue_phase<MT, true>(P, P.p1, sm, 0, seq);
            /* arrive at the grid barrier: the act rows of this CTA are stored */
            /* The lanes' act stores are ordered before lane 0's release by the warp barrier (release is
             * cumulative over it), so no lane needs a fence of its own. */
            __syncwarp();
            if (lane == 0) {
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.sync + 0) : "memory");
                stamp(P, 5);
            }
        }
        if (ok) ok = epilogue_phase<MT, false>(P, P.p2, sm, nt1, seq);
        if (lane == 0) stamp(P, 10);
        if (P.tp > 1) {
            /* every rank's partial sums of this CTA's rows arrive in this rank's own buffer as
             * tagged words (sent tile by tile during phase 2): wait for each, add in rank order */
            if (ok) {
                const unsigned long long *mine = P.peer_slots[P.rank] + (size_t)(seq & 1u) * P.tp * P.slot_stride;
                for (int i = lane; i < (e2 - b2) * MT; i += 32) {
                    const int row = b2 + i / MT, m = i % MT;
                    float a = 0.0f;
                    const bool all_in = tp_wait_sum(mine + (size_t)m * P.H + row, (size_t)P.slot_stride, P.tp, tp_tag(seq),
                                                    &sm->abort_flag, 20, &a);
                    if (!all_in) { give_up(sm, P.sync, ST_PEER_DATA); break; }
                    const float y = round_bf16(a);
                    P.out[(size_t)m * P.H + row] = f32_to_bf16_bits(y);
                    if (P.residual)
                        P.residual[(size_t)m * P.H + row] =
                            f32_to_bf16_bits(bf16_bits_to_f32(P.residual[(size_t)m * P.H + row]) + y);
                }
            }
            if (lane == 0) stamp(P, 11);
        }
    }
    __syncthreads();
    /* the call sequence number advances once per launch (parity of the peer slots, tag of the exchanged words) */
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (!P.gemv) P.sync[1] += gridDim.x; /* every CTA has arrived by now (this CTA passed the barrier) */
        if (P.tp > 1) atomicAdd(P.tp_seq, 1u);
        stamp(P, 12);
    }
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
    int overlap_ok = 0; /* dependent launch next to a cooperative one: 0 not tried yet, 1 taken, -1 refused */
};
static DeviceState g_dev[64];
static long long *g_trace = nullptr; /* debugging aid: device buffer for CTA 0's clock stamps */

void fused_set_trace(long long *device_buffer) { g_trace = device_buffer; }
long long *fused_get_trace() { return g_trace; }
static std::mutex g_dev_mutex;
static int g_launch_overlap = 1;
int fused_set_launch_overlap(int on) {
    const int old = g_launch_overlap;
    g_launch_overlap = on != 0;
    return old;
}

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

/* The whole geometry of a launch from the shape alone (no device needed): the two phases' thread
 * layouts and tiles, the stage size, how many stages the shared memory holds.  Pointers are left to
 * the caller.  Returns false when the kernel does not take the shape. */
static bool plan_fused(FusedParams &P, int tokens, int H, int I, int smem_optin, int target_bytes, int &c1, int &c2,
                       size_t &smem) {
    if (tokens < 1 || tokens > 2) return false;
    if (H <= 0 || I <= 0 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP) return false;
    if (H > (1 << 22) || I > (1 << 22)) return false; /* 32-bit row partitioning in the kernel */
    P.M = tokens; P.H = H; P.I = I;
    if (!plan_phase(P.p1, H, tokens, true, target_bytes, c1)) return false;
    if (!plan_phase(P.p2, I, tokens, false, target_bytes, c2)) return false;
    P.p1.rows_total = I; P.p1.up_offset = I;
    P.p2.rows_total = H; P.p2.up_offset = 0;
    const int part_floats = tokens == 1 ? kPartFloats1 : kPartFloats2;
    if (P.p1.TR * 2 * tokens * P.p1.nhw > part_floats || P.p2.TR * tokens * P.p2.nhw > part_floats) return false;
    P.stage_w_bytes = round_up(max(2 * P.p1.TR * P.p1.rb, P.p2.TR * P.p2.rb), 128);
    P.sc_half_bytes = round_up(max(P.p1.TR * P.p1.G * 2, P.p2.TR * P.p2.G * 2) + 32, 16);
    P.stage_bytes = round_up(P.stage_w_bytes + 2 * P.sc_half_bytes, 128);
    P.xs_bytes = round_up(tokens * I * 2, 128); /* act only: x is read from global memory */
    const size_t fixed = fused_smem_header(tokens) + (size_t)P.xs_bytes;
    if (fixed + 2 * (size_t)P.stage_bytes > (size_t)smem_optin) return false;
    P.nstages = (int)min((size_t)kMaxStages, ((size_t)smem_optin - fixed) / (size_t)P.stage_bytes);
    if (P.nstages < 2) return false;
    smem = fixed + (size_t)P.nstages * P.stage_bytes;
    return true;
}

template <int C1, int C2, int MT>
static int launch_fused(DeviceState &d, const FusedParams &P_in, int grid, size_t smem, cudaStream_t stream) {
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        bool &set = d.attr_set[C1 - 1][C2 - 1][MT - 1];
        if (!set) {
            FFN_CUDA_TRY(cudaFuncSetAttribute(ffn_fused_kernel<C1, C2, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              d.smem_optin), "fused FFN: shared-memory opt-in");
            set = true;
        }
    }
    FusedParams P = P_in;
    /* Programmatic dependent launch: consecutive launches in one stream overlap this launch's start
     * (CTA scheduling, barrier set-up, the first weight copies) with the tail of the one before.
     * Whether the driver takes the attribute next to a cooperative launch is found out once per
     * device, outside stream capture; until then, and wherever it is refused, the launch is the
     * plain cooperative one. */
    int overlap = 0;
    if (g_launch_overlap && !P.gemv) {
        if (d.overlap_ok == 1) {
            overlap = 1;
        } else if (d.overlap_ok == 0) {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) overlap = 2; /* probe */
        }
    }
    if (overlap) {
        P.early_weights = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attrs[2];
        attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[0].val.programmaticStreamSerializationAllowed = 1;
        attrs[1].id = cudaLaunchAttributeCooperative;
        attrs[1].val.cooperative = 1;
        cfg.attrs = attrs;
        cfg.numAttrs = 2;
        const cudaError_t err = cudaLaunchKernelEx(&cfg, ffn_fused_kernel<C1, C2, MT>, P);
        if (err == cudaSuccess) {
            if (overlap == 2) d.overlap_ok = 1;
            return FFN_OK;
        }
        if (overlap == 1) return fail(FFN_ERR_CUDA, "fused FFN launch: %s", cudaGetErrorString(err));
        (void)cudaGetLastError(); /* the probe was refused: remember, and launch the plain way */
        d.overlap_ok = -1;
        P.early_weights = 0;
    }
    void *args[] = {(void *)&P};
    FFN_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)ffn_fused_kernel<C1, C2, MT>, dim3(grid), dim3(kThreads),
                                             args, smem, stream), "fused FFN launch");
    return FFN_OK;
}

int fused_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                     const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual,
                     const FusedNorm *norm) {
    if (tokens < 1 || tokens > 4) return FFN_NOT_ADMITTED;
    DeviceState *dp = nullptr;
    const int st = device_state(&dp);
    if (st) return st;
    DeviceState &d = *dp;
    if (!d.cooperative) return FFN_NOT_ADMITTED;
    { /* a layer with a registered k-major copy of its down projection takes the kernel without the phase barrier */
        const bool with_norm = norm && norm->weight;
        FfnMlpWeights one = *w;
        if (with_norm) one.post_norm_w = norm->weight;
        const int km = kmajor_ffn_launch(stream, normed, act, layer_out, &one, 1, tokens, H, I, tp, residual, with_norm ? 1 : 0,
                                         with_norm ? norm->eps : 0.0f, with_norm ? norm->gemma : 0, d.sync + 3);
        if (km != FFN_NOT_ADMITTED) return km;
    }
    if (tokens > 2) return FFN_NOT_ADMITTED; /* the row-major single-launch kernel takes one or two tokens */
    if (((uintptr_t)w->gate_up_i4 & 15) || ((uintptr_t)w->down_i4 & 15) || ((uintptr_t)normed & 15) ||
        ((uintptr_t)act & 15) || ((uintptr_t)w->gate_up_i4_scales & 15) || ((uintptr_t)w->down_i4_scales & 15))
        return FFN_NOT_ADMITTED;

    FusedParams P = {};
    P.x = (const uint16_t *)normed;
    P.act = (uint16_t *)act;
    P.out = (uint16_t *)layer_out;
    P.M = tokens; P.H = H; P.I = I;
    P.sync = d.sync;
    P.tp = 1; P.rank = 0;
    P.residual = (uint16_t *)residual;
    if (norm && norm->weight) {
        if ((uintptr_t)norm->weight & 15) return FFN_NOT_ADMITTED;
        P.norm_w = (const uint16_t *)norm->weight; P.norm_eps = norm->eps; P.norm_gemma = norm->gemma;
    }
    if (tp && tp->tp > 1) {
        P.tp = tp->tp; P.rank = tp->rank;
        P.peer_slots = tp->peer_slots; P.slot_stride = tp->slot_stride;
        P.tp_seq = tp->seq;
        if (tokens * H > tp->slot_stride) return fail(FFN_ERR_CONFIG, "fused FFN: %d tokens exceed the exchange buffer", tokens);
    }
#ifdef FFN_INT4_TUNING
    static const int target_kb = getenv("FFN_INT4_STAGE_KB") ? atoi(getenv("FFN_INT4_STAGE_KB")) : kDefaultStageTarget / 1024;
#else
    const int target_kb = kDefaultStageTarget / 1024;
#endif
    int c1 = 0, c2 = 0;
    size_t smem = 0;
    if (!plan_fused(P, tokens, H, I, d.smem_optin, target_kb * 1024, c1, c2, smem)) return FFN_NOT_ADMITTED;
    P.p1.w = w->gate_up_i4; P.p1.s = (const uint16_t *)w->gate_up_i4_scales;
    P.p2.w = w->down_i4; P.p2.s = (const uint16_t *)w->down_i4_scales;
    P.trace = g_trace;
#ifdef FFN_INT4_TUNING
    static const int debug_flags = getenv("FFN_INT4_DEBUG") ? atoi(getenv("FFN_INT4_DEBUG")) : 0;
    P.debug = debug_flags;
#endif
    const int grid = d.sm_count; /* under TP every rank runs the same grid: CTA c owns the same rows everywhere */

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
    return fused_ffn_launch(stream, normed, act, layer_out, w, tokens, H, I, nullptr, nullptr, nullptr);
}

/* ------------------------------------------------------------------------------------------- */
/* The fused FFN for callers that cannot allocate                                               */
/* ------------------------------------------------------------------------------------------- */
/* Some hosts give every byte of device memory to an arena of their own when they start, so a later
 * cudaMalloc from inside a library fails; others run the decode loop in a place where the implicit
 * device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.  For them the scratch the
 * fused kernel needs besides its inputs and outputs - the four synchronisation words and the
 * activation vector act = SiLU(gate)*up that phase 1 hands to phase 2 through global memory - lives
 * in this fixed array instead of in allocated memory.  Every GPU that loads the library holds these
 * 128.25 KiB until the process exits.  Limit: tokens * intermediate_size <= kNoAllocActElems. */
constexpr int kNoAllocActElems = 65536;                              /* bf16 elements of act */
constexpr size_t kNoAllocSyncBytes = 256;
constexpr size_t kNoAllocBytes = kNoAllocSyncBytes + (size_t)kNoAllocActElems * 2;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

/* Per device: the DEVICE address of the array above.  In host code the name g_noalloc_scratch is
 * only a stand-in for the symbol; the address a kernel can use comes from cudaGetSymbolAddress,
 * asked once per device with that device current. */
static DeviceState g_noalloc_dev[64];
static unsigned char *g_noalloc_ptr[64];

static int noalloc_device_state(DeviceState **out, unsigned char **scratch) {
    int dev = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FFN_ERR_CONFIG, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState &d = g_noalloc_dev[dev];
    if (!d.ready) {
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev), "SM count");
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "smem opt-in");
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.cooperative, cudaDevAttrCooperativeLaunch, dev), "cooperative launch");
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(FFN_ERR_CUDA, "cannot resolve the static scratch array on device %d: %s", dev, cudaGetErrorString(e));
        g_noalloc_ptr[dev] = (unsigned char *)p;
        d.sync = (unsigned *)p; /* the first kNoAllocSyncBytes of the array */
        d.ready = true;
    }
    *out = &d;
    *scratch = g_noalloc_ptr[dev];
    return FFN_OK;
}

int fused_ffn_launch_noalloc(cudaStream_t stream, const void *normed, void *layer_out,
                             const FfnMlpWeights *w, int tokens, int H, int I) {
    if (tokens < 1 || tokens > 2)
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: %d tokens; this entry point takes 1 or 2", tokens);
    if (H > (1 << 22)) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: hidden size %d is beyond the kernel's range", H);
    if ((long long)tokens * I > kNoAllocActElems)
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: tokens * intermediate_size = %lld exceeds the "
                    "static scratch (%d elements)", (long long)tokens * I, kNoAllocActElems);
    DeviceState *dp = nullptr;
    unsigned char *scratch = nullptr;
    const int st = noalloc_device_state(&dp, &scratch);
    if (st) return st;
    DeviceState &d = *dp;
    if (!d.cooperative) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: the device cannot launch cooperatively");
    if (((uintptr_t)w->gate_up_i4 & 15) || ((uintptr_t)w->down_i4 & 15) || ((uintptr_t)normed & 15) ||
        ((uintptr_t)w->gate_up_i4_scales & 15) || ((uintptr_t)w->down_i4_scales & 15))
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: operands must be 16-byte aligned");

    FusedParams P = {};
    P.x = (const uint16_t *)normed;
    P.act = (uint16_t *)(scratch + kNoAllocSyncBytes);
    P.out = (uint16_t *)layer_out;
    P.M = tokens; P.H = H; P.I = I;
    P.sync = d.sync;
    P.tp = 1; P.rank = 0;
    int c1 = 0, c2 = 0;
    size_t smem = 0;
    if (!plan_fused(P, tokens, H, I, d.smem_optin, kDefaultStageTarget, c1, c2, smem))
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: rows of %d / %d columns do not fit the kernel's "
                    "shared memory", H, I);
    P.p1.w = w->gate_up_i4; P.p1.s = (const uint16_t *)w->gate_up_i4_scales;
    P.p2.w = w->down_i4; P.p2.s = (const uint16_t *)w->down_i4_scales;
    /* The array keeps whatever the previous call left.  The barrier words must be consistent with
     * each other, so they are cleared on the stream first; act needs no clearing (phase 1 writes
     * every element phase 2 reads).  The status word (word 3) is NOT cleared here: a wait that ran
     * out in an earlier call stays on record until ffn_int4_noalloc_status reads it. */
    FFN_CUDA_TRY(cudaMemsetAsync(d.sync, 0, 3 * sizeof(unsigned), stream), "clear the static synchronisation words");
    const int grid = d.sm_count;
    if (tokens == 1) {
        if (c1 == 1 && c2 == 1) return launch_fused<1, 1, 1>(d, P, grid, smem, stream);
        if (c1 == 1 && c2 == 2) return launch_fused<1, 2, 1>(d, P, grid, smem, stream);
        if (c1 == 2 && c2 == 1) return launch_fused<2, 1, 1>(d, P, grid, smem, stream);
        return launch_fused<2, 2, 1>(d, P, grid, smem, stream);
    }
    return launch_fused<1, 1, 2>(d, P, grid, smem, stream);
}

/* Text description of what a launch of this shape would look like on a device with `sm_count` SMs
 * and `smem_optin` bytes of opt-in shared memory; needs no device.  Returns false when the kernel
 * does not take the shape. */
bool fused_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes) {
    FusedParams P = {};
    int c1 = 0, c2 = 0;
    size_t smem = 0;
    if (!plan_fused(P, tokens, H, I, smem_optin, kDefaultStageTarget, c1, c2, smem)) return false;
    snprintf(out, out_bytes,
             "kernel=fused grid=%d threads=%d smem=%zu stages=%d stage_bytes=%d act_bytes=%d "
             "p1_cit=%d p1_ct=%d p1_rg=%d p1_jt=%d p1_pairs_per_tile=%d p2_cit=%d p2_ct=%d p2_rg=%d p2_jt=%d p2_rows_per_tile=%d",
             sm_count, kThreads, smem, P.nstages, P.stage_bytes, P.xs_bytes, c1, P.p1.CT, P.p1.RG, P.p1.JT, P.p1.TR, c2,
             P.p2.CT, P.p2.RG, P.p2.JT, P.p2.TR);
    return true;
}

int fused_status_word(unsigned **out) {
    DeviceState *dp = nullptr;
    const int st = device_state(&dp);
    if (st) return st;
    *out = dp->sync + 3;
    return FFN_OK;
}

/* The status word of the static-scratch entry point on the current device (no allocation: the
 * array's address is looked up, the four words are copied to the host).  A device that never ran
 * that entry point and has not resolved the array yet is resolved here. */
int fused_status_noalloc(unsigned *status_out, bool reset) {
    DeviceState *dp = nullptr;
    unsigned char *scratch = nullptr;
    const int st = noalloc_device_state(&dp, &scratch);
    if (st) return st;
    unsigned words[4];
    FFN_CUDA_TRY(cudaMemcpy(words, dp->sync, sizeof(words), cudaMemcpyDeviceToHost), "read the static status word");
    *status_out = words[3];
    if (reset && words[3] != 0) FFN_CUDA_TRY(cudaMemset(dp->sync, 0, sizeof(words)), "reset the static synchronisation words");
    return FFN_OK;
}

/* True once the static array has been resolved on the current device (i.e. the allocation-free
 * entry point or its status reader ran there). */
bool fused_noalloc_in_use() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    return g_noalloc_dev[dev].ready;
}

int fused_status(unsigned *status_out, bool reset) {
    DeviceState *dp = nullptr;
    const int st = device_state(&dp);
    if (st) return st;
    unsigned words[4];
    FFN_CUDA_TRY(cudaMemcpy(words, dp->sync, sizeof(words), cudaMemcpyDeviceToHost), "read kernel status");
    *status_out = words[3];
    if (reset && words[3] != 0) {
        FFN_CUDA_TRY(cudaMemset(dp->sync, 0, sizeof(words)), "reset synchronisation words");
        kmajor_reset_sync();
        tc_reset_sync();
    }
    return FFN_OK;
}

/* Geometry of a single-matrix launch (out[M][N] = a[M][K] x W[N][K]^T): the kernel's second phase
 * alone, its activation vector being the caller's input.  Returns false when the kernel does not
 * take the shape. */
static bool plan_gemv(FusedParams &P, int tokens, int N, int K, int smem_optin, int target_bytes, int &c2, size_t &smem) {
    if (tokens < 1 || tokens > 2) return false;
    if (N <= 0 || K <= 0 || K % FFN_INT4_GROUP || N % 8) return false; /* N % 8: the scale array ends on a 16-byte boundary */
    if (N > (1 << 22) || K > (1 << 22)) return false;
    P.M = tokens; P.H = N; P.I = K;
    P.gemv = 1;
    P.p1 = PhasePlan();
    P.p1.TR = 1; /* no rows: zero tiles */
    if (!plan_phase(P.p2, K, tokens, false, target_bytes, c2)) return false;
    P.p2.rows_total = N; P.p2.up_offset = 0;
    const int part_floats = tokens == 1 ? kPartFloats1 : kPartFloats2;
    if (P.p2.TR * tokens * P.p2.nhw > part_floats) return false;
    P.stage_w_bytes = round_up(P.p2.TR * P.p2.rb, 128);
    P.sc_half_bytes = round_up(P.p2.TR * P.p2.G * 2 + 32, 16);
    P.stage_bytes = round_up(P.stage_w_bytes + P.sc_half_bytes, 128);
    P.xs_bytes = 0; /* the consumers read their slices of the activation straight from global memory */
    const size_t fixed = fused_smem_header(tokens) + (size_t)P.xs_bytes;
    if (fixed + 2 * (size_t)P.stage_bytes > (size_t)smem_optin) return false;
    P.nstages = (int)min((size_t)kMaxStages, ((size_t)smem_optin - fixed) / (size_t)P.stage_bytes);
    smem = fixed + (size_t)P.nstages * P.stage_bytes;
    return true;
}

/* One or two activation rows against one packed matrix through the streaming kernel (persistent
 * CTA per SM, bulk-copy ring, dp4a inner product): the replacement for gemv_int4_kernel
 * (csrc/kernels/gemm_quant.cu:165-200) on its own, i.e. for projections and the LM head as well as
 * for the FFN's two matrices.  FFN_NOT_ADMITTED when the shape or the alignment is outside what the
 * kernel takes. */
static int gemv_int4_stream(const void *a, const void *packed, const void *scales, void *out, int M, int N, int K,
                            cudaStream_t stream) {
    if (M < 1 || M > 2) return FFN_NOT_ADMITTED;
    if (((uintptr_t)a & 15) || ((uintptr_t)packed & 15) || ((uintptr_t)scales & 15)) return FFN_NOT_ADMITTED;
    DeviceState *dp = nullptr;
    const int st = device_state(&dp);
    if (st) return st;
    DeviceState &d = *dp;
    if (!d.cooperative) return FFN_NOT_ADMITTED;
    FusedParams P = {};
    int c2 = 0;
    size_t smem = 0;
    if (!plan_gemv(P, M, N, K, d.smem_optin, kDefaultStageTarget, c2, smem)) return FFN_NOT_ADMITTED;
    P.x = (const uint16_t *)a;
    P.act = nullptr; /* nothing is handed over between phases */
    P.out = (uint16_t *)out;
    P.sync = d.sync;
    P.tp = 1; P.rank = 0;
    P.p2.w = (const uint8_t *)packed; P.p2.s = (const uint16_t *)scales;
    P.trace = nullptr;
    const int grid = min(d.sm_count, (N + P.p2.TR - 1) / P.p2.TR); /* no CTA without a tile */
    if (M == 2) return launch_fused<1, 1, 2>(d, P, grid, smem, stream);
    if (c2 == 1) return launch_fused<1, 1, 1>(d, P, grid, smem, stream);
    return launch_fused<1, 2, 1>(d, P, grid, smem, stream);
}

bool gemv_describe_plan(int tokens, int N, int K, int sm_count, int smem_optin, char *out, size_t out_bytes) {
    FusedParams P = {};
    int c2 = 0;
    size_t smem = 0;
    if (!plan_gemv(P, tokens, N, K, smem_optin, kDefaultStageTarget, c2, smem)) return false;
    snprintf(out, out_bytes, "kernel=stream_gemv grid=%d threads=%d smem=%zu stages=%d stage_bytes=%d x_bytes=%d cit=%d ct=%d rg=%d jt=%d rows_per_tile=%d",
             min(sm_count, (N + P.p2.TR - 1) / P.p2.TR), kThreads, smem, P.nstages, P.stage_bytes, P.xs_bytes, c2, P.p2.CT, P.p2.RG,
             P.p2.JT, P.p2.TR);
    return true;
}

int gemm_int4_dispatch(const void *a, const void *packed, const void *scales, void *out, int M, int N,
                       int K, cudaStream_t stream) {
    if (M <= 2) {
        const int st = gemv_int4_stream(a, packed, scales, out, M, N, K, stream);
        if (st != FFN_NOT_ADMITTED) return st;
    }
    return gemm_int4_generic(a, packed, scales, out, nullptr, M, N, K, stream);
}

}  // namespace ffn
