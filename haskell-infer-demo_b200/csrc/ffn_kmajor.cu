/*
 * ffn_kmajor.cu - the decode-shaped (M <= 2) INT4 FFN, one or many layers, as ONE persistent kernel
 * whose second projection needs no grid-wide hand-over of the activation vector.
 *
 * The row-major single-launch kernel (ffn_fused.cu) has to stop between its phases: a down-projection
 * row needs the whole act vector, so every CTA waits at a grid barrier, fetches act and converts it
 * again - a bubble of several microseconds during which the weight stream is only kept alive by
 * prefetch.  Here CTA c multiplies the down projection against ONLY the act values it produced
 * itself (its 8-aligned K range of about I/148 elements), for ALL output rows.  With the reference's
 * row-major [H][I/2] layout that would be a 59-byte sliver of every row; with a k-major copy of the
 * matrix - WT[I/8][H] 32-bit words, word (kb, h) = the eight codes k = 8kb..8kb+7 of output row h, and
 * ST[I/128][H] scales - it is a few contiguous 4H-byte rows, streamed through the same bulk-copy ring
 * as the gate/up rows.  act never leaves the CTA (it is still written to the caller's workspace), the
 * eight activations of a k-block are uniform across the CTA (byte planes broadcast from shared
 * memory), the integer sums need no cross-thread reduction, and phase 2 starts the moment the CTA's
 * own phase-1 epilogue is done.  What remains is a sum over CTAs: every CTA leaves FP32 partial sums
 * for all H rows in global memory and then adds, in CTA order, the partials of the ~H/148 rows it owns.
 *
 * Nothing in that hand-over uses a fence or a flag: a partial sum travels as one 8-byte word {value,
 * tag of this layer} and the reader polls the word itself (the protocol of the cross-rank exchange,
 * kernels.h).  A relaxed arrival counter only tells the readers when polling is worth starting.  The
 * same holds for the residual stream between the layers of a stack: the CTA that owns a row publishes
 * the updated h as a tagged word, and the loader threads of every CTA pick the next layer's input up
 * from those words.  One launch therefore runs any number of layers (the producer warp simply keeps
 * streaming the next layer's rows while the epilogues and the cross-rank exchange of the current one
 * are in flight), replacing per layer the reference's norm + three kernels + leader all-reduce +
 * residual add (csrc/kernels/layers.cu:127-160; csrc/engine.cu:1603-1657; csrc/collective.cu:168-219).
 *
 * Roles (one CTA per SM, 19 warps, as in ffn_fused.cu): warp 0 producer, warps 1..17 consumers
 * (phase 1: half-warp dot products over gate/up row pairs; phase 2: per-thread output columns over
 * the k-major rows; then the reduce over CTAs, the cross-rank exchange, output and residual update),
 * warp 18 the phase-1 epilogue (rounding points, SiLU*up, byte planes of the CTA's act values).
 *
 * Every device-side wait is bounded; on expiry the kernel records where it gave up, drains its own
 * copies and returns.
 */
#include <stdio.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "kernels.h"
#include "stream_common.cuh"
#include "kmajor_common.cuh"

namespace ffn {

constexpr int kKmMaxLayers = 64;      /* layers per launch (their pointers travel in the kernel parameters) */
constexpr int kKmMaxKb = 32;          /* k-blocks (8 act values each) one CTA may own */
constexpr int kKmMaxSeg = 3;          /* 128-groups such a range can touch */
constexpr int kKmMaxPairs = 6;        /* output column pairs per consumer thread: H <= 2 * 544 * 6 */
constexpr int kKmMaxQ = 20;           /* partial sums one reducer lane adds: grid <= 8 * 20 */
constexpr int kKmGroupKb = FFN_INT4_GROUP / 8; /* k-blocks per scale group */

struct KmLayer {
    const uint8_t *gu_w;      /* gate/up pair, row-major [2I][H/2] */
    const uint16_t *gu_s;     /* its scales [2I][H/128] */
    const uint32_t *wt;       /* k-major down projection [I/8][H] */
    const uint16_t *st;       /* its scales [I/128][H] */
    const uint16_t *norm_w;   /* RMSNorm weight of this layer's input, or NULL */
};

struct KmParams {
    const uint16_t *x;        /* [M][H] bf16: input of the first layer (already normalized, or the residual stream h) */
    uint16_t *act;            /* [M][I] bf16 in the caller's workspace (the last layer's act is what remains) */
    uint16_t *out;            /* [M][H] bf16: the reduced FFN output (of the last layer) */
    uint16_t *residual;       /* optional h <- bf16(h + y); in a stack this is x itself */
    int residual_is_x;        /* the residual stream is the kernel's input (its current value is in shared memory) */
    int M, H, I, L;
    PhasePlan p1;             /* gate/up tiling (w, s unused: per layer) */
    int R2;                   /* k-major rows per phase-2 tile */
    int stage_bytes, nstages, stage_w_bytes, sc_half_bytes, xs_bytes;
    unsigned *sync;           /* [0] arrivals "partials stored", [1] arrivals "h published", [2] both counters'
                                 value when this launch began, [3] layers run so far (the base of the tags) */
    unsigned *status;         /* the device's kernel status word */
    unsigned long long *partial; /* [grid][M][H] tagged words */
    unsigned long long *hx;      /* [M][H] tagged words: the residual stream between layers */
    /* tensor parallelism (tp == 1: unused) */
    int tp, rank, slot_stride;
    unsigned long long *const *peer_slots;
    unsigned *tp_seq;
    float norm_eps;
    int norm_gemma;
    long long *trace;
    KmLayer layers[kKmMaxLayers];
};

struct KmSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t part_full[kPartSlots];
    uint64_t part_empty[kPartSlots];
    uint64_t x_ready;         /* the layer's input is staged in shared memory (loader warps arrive) */
    uint64_t act_ready;       /* this CTA's act values and their byte planes are in place (epilogue arrives) */
    uint64_t p_open;          /* every CTA has stored this layer's partial sums (the epilogue warp saw the counter) */
    uint64_t h_open;          /* every CTA has published this layer's residual rows (likewise) */
    unsigned arrive_p, arrive_h; /* consumer warps of this CTA that finished storing / publishing (monotonic) */
    int abort_flag;
    unsigned base;            /* the arrival counters' value when the launch began */
    unsigned epoch;           /* layers this device has run before this launch: layer l's words carry km_tag(epoch + l) */
    unsigned seq0;            /* the communicator's call number when the launch began */
    int pad[2];
    float norm_red[2][kConsumerWarps + 3];
    float fac[2][kKmMaxSeg + 1];
    __align__(16) uint32_t planes[2][kKmMaxKb][4];   /* [token][k-block]{he, ho, le, lo} */
    uint16_t act_s[2][kKmMaxKb * 8];   /* this CTA's act values */
    float part[1];            /* kPartSlots slots of kPartFloats1 or kPartFloats2 floats follow */
};

__host__ __device__ constexpr size_t km_smem_header(int tokens) {
    return (sizeof(KmSmem) + (size_t)kPartSlots * (tokens == 1 ? kPartFloats1 : kPartFloats2) * sizeof(float) + 127) / 128 * 128;
}

__device__ __forceinline__ void km_give_up(KmSmem *sm, unsigned *status, int where) {
    sm->abort_flag = 1;
    atomicCAS(status, 0u, (unsigned)where | ((unsigned)blockIdx.x << 8));
}
/* Optional timeline: 16 stamps per CTA of the global nanosecond timer (comparable across SMs). */
__device__ __forceinline__ void km_stamp(const KmParams &P, int slot) {
    if (P.trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        P.trace[(size_t)blockIdx.x * 16 + slot] = (long long)t;
    }
}
/* The four byte planes of eight block-fixed-point activations X[0..7] (16-bit two's complement in the
 * low halves), laid out for chunk_dot-style dp4a against one widened weight word: he / le pair with
 * the even codes, ho / lo with the odd ones (the layout prepare_chunk builds, stream_common.cuh). */
__device__ __forceinline__ uint4 km_planes(const int (&X)[8]) {
    const uint32_t e02 = prmt(X[0], X[2], 0x5140), e46 = prmt(X[4], X[6], 0x5140);
    const uint32_t o13 = prmt(X[1], X[3], 0x5140), o57 = prmt(X[5], X[7], 0x5140);
    uint4 p;
    p.x = prmt(e02, e46, 0x7632); /* he */
    p.y = prmt(o13, o57, 0x7632); /* ho */
    p.z = prmt(e02, e46, 0x5410); /* le */
    p.w = prmt(o13, o57, 0x5410); /* lo */
    return p;
}

/* ---- producer: the weight stream of all layers ------------------------------------------------ */
__device__ __forceinline__ void km_producer(const KmParams &P, KmSmem *sm, uint8_t *ring, int kb0, int kb1) {
    const int ns = P.nstages;
    const int nkb = kb1 - kb0;
    const int pair0 = kb0 * 8, pair1 = kb1 * 8;
    const int nt1 = (pair1 - pair0 + P.p1.TR - 1) / P.p1.TR;
    const int nt2 = (nkb + P.R2 - 1) / P.R2;
    const uint32_t row2 = (uint32_t)P.H * 4u;
    int t = 0;
    bool failed = false;
    for (int l = 0; l < P.L && !failed; ++l) {
        const KmLayer &LY = P.layers[l];
        for (int lt = 0; lt < nt1 + nt2; ++lt, ++t) {
            const int s = t % ns;
            if (t >= ns && !mbar_wait<100>(&sm->empty[s], (uint32_t)(t / ns - 1) & 1u, &sm->abort_flag)) {
                km_give_up(sm, P.status, ST_PRODUCER_EMPTY);
                failed = true;
                break;
            }
            uint8_t *dst = ring + (size_t)s * P.stage_bytes;
            if (lt < nt1) {
                const int r0 = pair0 + lt * P.p1.TR, rows = min(P.p1.TR, pair1 - r0);
                const uint32_t bytes = (uint32_t)rows * P.p1.rb;
                /* scale runs widened to 16-byte boundaries (the array's end is one: row counts are
                 * multiples of 8, so N*G*2 is a multiple of 16) */
                const size_t g0 = (size_t)r0 * P.p1.G * 2, g1 = (size_t)(r0 + P.p1.up_offset) * P.p1.G * 2;
                const size_t len = (size_t)rows * P.p1.G * 2;
                const size_t a0 = g0 & ~(size_t)15, a1 = g1 & ~(size_t)15;
                const uint32_t n0 = (uint32_t)(((g0 + len + 15) & ~(size_t)15) - a0);
                const uint32_t n1 = (uint32_t)(((g1 + len + 15) & ~(size_t)15) - a1);
                mbar_expect_tx(&sm->full[s], 2 * bytes + n0 + n1);
                bulk_g2s(dst, LY.gu_w + (size_t)r0 * P.p1.rb, bytes, &sm->full[s]);
                bulk_g2s(dst + bytes, LY.gu_w + (size_t)(r0 + P.p1.up_offset) * P.p1.rb, bytes, &sm->full[s]);
                bulk_g2s(dst + P.stage_w_bytes, (const uint8_t *)LY.gu_s + a0, n0, &sm->full[s]);
                bulk_g2s(dst + P.stage_w_bytes + P.sc_half_bytes, (const uint8_t *)LY.gu_s + a1, n1, &sm->full[s]);
            } else {
                const int r0 = kb0 + (lt - nt1) * P.R2, rows = min(P.R2, kb1 - r0);
                const uint32_t bytes = (uint32_t)rows * row2;
                mbar_expect_tx(&sm->full[s], bytes);
                bulk_g2s(dst, LY.wt + (size_t)r0 * P.H, bytes, &sm->full[s]);
            }
        }
    }
    /* Never leave with a copy of ours still in flight: wait (bounded) for the most recent fill of every stage. */
    for (int u = max(0, t - ns); u < t; ++u) {
        bool done = false;
        for (uint32_t i = 0; i < kSpinLimit && !done; ++i) done = mbar_try_wait(&sm->full[u % ns], (uint32_t)(u / ns) & 1u);
        if (!done) atomicCAS(P.status, 0u, (unsigned)ST_DRAIN | ((unsigned)blockIdx.x << 8));
    }
}

/* ---- epilogue warp: phase-1 sums -> act, then the byte planes of this CTA's act values --------- */
template <int MT>
__device__ __forceinline__ bool km_epilogue_layer(const KmParams &P, KmSmem *sm, int l, int kb0, int kb1, int part_tile0, unsigned &base) {
    constexpr int NVROW = 2 * MT;
    const PhasePlan &pl = P.p1;
    const int lane = threadIdx.x & 31;
    const int pair0 = kb0 * 8, pair1 = kb1 * 8;
    const int ntiles = (pair1 - pair0 + pl.TR - 1) / pl.TR;
    if (l == 0) {
        /* Both arrival counters stood at `base` when the launch began; `epoch` numbers the layers this
         * device has run (the tags); seq0 is the communicator's call number.  Stable until CTA 0 rewrites
         * them at its exit, which it reaches only after every CTA has arrived at the last layer's
         * counters.  Read here, off everybody's critical path, and published to the consumers by this
         * warp's arrivals at act_ready / p_open. */
        unsigned b = 0;
        if (lane == 0) {
            b = P.sync[2];
            sm->base = b;
            sm->epoch = P.sync[3];
            sm->seq0 = P.tp > 1 ? ld_acquire_gpu(P.tp_seq) : 0u;
        }
        base = __shfl_sync(0xffffffffu, b, 0);
    }
    for (int lt = 0; lt < ntiles; ++lt) {
        const int pt = part_tile0 + lt;
        const int pslot = pt % kPartSlots;
        const int rows = min(pl.TR, pair1 - (pair0 + lt * pl.TR));
        if (!mbar_wait<100>(&sm->part_full[pslot], (uint32_t)(pt / kPartSlots) & 1u, &sm->abort_flag)) {
            km_give_up(sm, P.status, ST_PART_FULL);
            return false;
        }
        const float *part = sm->part + (size_t)pslot * (MT == 1 ? kPartFloats1 : kPartFloats2);
        for (int i = lane; i < rows * MT; i += 32) {
            const int p = i / MT, m = i % MT;
            const int row = pair0 + lt * pl.TR + p;
            float a = 0.0f, b = 0.0f;
            const float *pa = part + ((size_t)p * NVROW + m) * pl.nhw;
            const float *pb = part + ((size_t)p * NVROW + MT + m) * pl.nhw;
#pragma unroll 4
            for (int h = 0; h < pl.nhw; ++h) a += pa[h];
#pragma unroll 4
            for (int h = 0; h < pl.nhw; ++h) b += pb[h];
            const uint16_t v = f32_to_bf16_bits(silu_mul(round_bf16(a), round_bf16(b)));
            P.act[(size_t)m * P.I + row] = v;
            sm->act_s[m][row - pair0] = v;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->part_empty[pslot]);
    }
    __syncwarp();
    /* Block fixed point with one exponent per (token, 128-group segment of this CTA's K range):
     * X_k = rint(a_k * 2^(14-E)), E = exponent of the segment's largest magnitude.  A segment that
     * holds an Inf or a NaN gets fac = NaN, so every output of that token becomes NaN. */
    const int nseg = kb1 > kb0 ? (kb1 - 1) / kKmGroupKb - kb0 / kKmGroupKb + 1 : 0;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        for (int seg = 0; seg < nseg; ++seg) {
            const int g = kb0 / kKmGroupKb + seg;
            const int lo = max(kb0, g * kKmGroupKb), hi = min(kb1, (g + 1) * kKmGroupKb);
            uint32_t mx = 0;
            for (int e = (lo - kb0) * 8 + lane; e < (hi - kb0) * 8; e += 32) mx = max(mx, (uint32_t)(sm->act_s[m][e] & 0x7FFFu));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const int E = (int)(mx >> 7);
            const bool live = E >= 19 && E < 255;
            const float up = live ? __uint_as_float((uint32_t)(268 - E) << 23) : 0.0f;
            if (lane == 0)
                sm->fac[m][seg] = live ? __uint_as_float((uint32_t)(E - 18) << 23) : (E == 255 ? __uint_as_float(0x7FC00000u) : 0.0f);
            const int kb = lo + lane;
            if (kb < hi) {
                int X[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    X[i] = __float_as_int(fmaf(bf16_bits_to_f32(sm->act_s[m][(kb - kb0) * 8 + i]), up, 12582912.0f));
                *(uint4 *)sm->planes[m][kb - kb0] = km_planes(X);
            }
        }
    }
    __syncwarp();
    if (lane == 0 && kb1 > kb0) { /* a CTA without k-blocks has no act: its consumers do not wait for any */
        mbar_arrive(&sm->act_ready);
        if (l == 0) km_stamp(P, 5);
    }
    /* From here on this warp is idle until the next layer, so it watches the two arrival counters for
     * the whole CTA (one poller per SM): when every CTA has stored its partial sums the reducers may
     * start reading them, when every CTA has published its rows of h the loaders may.  Hints only -
     * the words validate themselves. */
    bool ok = true;
    if (lane == 0) {
        const unsigned target = base + (unsigned)(l + 1) * gridDim.x;
        ok = km_wait_counter(P.sync + 0, target, &sm->abort_flag);
        if (ok) {
            mbar_arrive(&sm->p_open);
            if (l == 0) km_stamp(P, 13);
            if (l + 1 < P.L) {
                ok = km_wait_counter(P.sync + 1, target, &sm->abort_flag);
                if (ok) mbar_arrive(&sm->h_open);
            }
        }
        if (!ok) km_give_up(sm, P.status, ST_PARTIALS);
    }
    return __shfl_sync(0xffffffffu, ok, 0);
}

/* ---- consumers: staging of the layer's input ---------------------------------------------------- */
/* The loader threads (row group 0 of the phase-1 layout: one thread per 32-element column chunk)
 * bring the layer's input into shared memory - from the caller's buffer for the first layer, from the
 * tagged words the previous layer's owners published for the others - and leave the sums of squares
 * for the fused RMSNorm.  Returns false when a wait ran out. */
/* The first layer's input is in place when the kernel starts: the loader threads fetch their slices
 * before anything else happens (before the producer has filled the memory system with bulk copies,
 * behind which a load issued later would queue for microseconds). */
template <int CIT, int MT>
__device__ __forceinline__ void km_prefetch_input(const KmParams &P, uint32_t (&pre)[CIT][MT][16]) {
    const PhasePlan &pl = P.p1;
    const int ti = threadIdx.x - 32;
#pragma unroll
    for (int c = 0; c < CIT; ++c)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int col = ti + c * pl.CT;
            const bool on = ti >= 0 && ti < pl.CT && col < pl.cpr;
            const uint16_t *src = P.x + (size_t)m * pl.K + (size_t)(on ? col : 0) * 32;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 t4 = make_uint4(0, 0, 0, 0);
                if (on) t4 = __ldg((const uint4 *)(src + q * 8));
                pre[c][m][4 * q] = t4.x; pre[c][m][4 * q + 1] = t4.y; pre[c][m][4 * q + 2] = t4.z; pre[c][m][4 * q + 3] = t4.w;
            }
        }
}

/* ... and put them into shared memory as soon as the barriers exist, with the sums of squares for a
 * fused RMSNorm, exactly as km_stage_input does for the later layers. */
template <int CIT, int MT>
__device__ __forceinline__ void km_stage_first(const KmParams &P, KmSmem *sm, uint16_t *xs, const uint32_t (&pre)[CIT][MT][16]) {
    const PhasePlan &pl = P.p1;
    const int ti = threadIdx.x - 32, lane = threadIdx.x & 31, wp = ti >> 5;
    if (ti < 0 || wp >= (pl.CT + 31) / 32) return;
    float ss[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) ss[m] = 0.0f;
#pragma unroll
    for (int c = 0; c < CIT; ++c) {
        const int col = ti + c * pl.CT;
        if (ti >= pl.CT || col >= pl.cpr) continue;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint32_t *dst = (uint32_t *)(xs + (size_t)m * pl.K + (size_t)col * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q)
                *(uint4 *)(dst + 4 * q) = make_uint4(pre[c][m][4 * q], pre[c][m][4 * q + 1], pre[c][m][4 * q + 2], pre[c][m][4 * q + 3]);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                ss[m] = fmaf(bf16_lo(pre[c][m][q]), bf16_lo(pre[c][m][q]), ss[m]);
                ss[m] = fmaf(bf16_hi(pre[c][m][q]), bf16_hi(pre[c][m][q]), ss[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float tot = warp_sum(ss[m]);
        if (lane == 0) sm->norm_red[m][wp] = tot;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->x_ready);
}

template <int CIT, int MT>
__device__ __forceinline__ bool km_stage_input(const KmParams &P, KmSmem *sm, uint16_t *xs, int l) {
    if (l == 0) return true; /* staged by km_stage_first */
    const PhasePlan &pl = P.p1;
    const int ti = threadIdx.x - 32, lane = threadIdx.x & 31, wp = ti >> 5;
    const int loader_warps = (pl.CT + 31) / 32;
    if (wp >= loader_warps) return true;
    const bool loader = ti < pl.CT;
    if (!mbar_wait<64>(&sm->h_open, (uint32_t)(l - 1) & 1u, &sm->abort_flag)) {
        /* (the epilogue warp watches the arrival counter for the whole CTA: one poller per SM) */
        if (lane == 0) km_give_up(sm, P.status, ST_NEXT_X);
        return false;
    }
    const unsigned tag = km_tag(sm->epoch + (unsigned)l - 1u); /* the previous layer's */
    float ss[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) ss[m] = 0.0f;
    bool bad = false;
#pragma unroll
    for (int c = 0; c < CIT; ++c) {
        const int col = ti + c * pl.CT;
        if (!loader || col >= pl.cpr) continue;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint32_t v[16];
            {
                const unsigned long long *src = P.hx + (size_t)m * pl.K + (size_t)col * 32;
                bool in = false;
                for (uint32_t k = 0; k < kTpPollLimit && !in; ++k) {
                    in = true;
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        unsigned long long a, b;
                        km_load2(src + 2 * q, a, b);
                        in = in && (unsigned)(a >> 32) == tag && (unsigned)(b >> 32) == tag;
                        v[q] = ((unsigned)a >> 16) | ((unsigned)b & 0xFFFF0000u); /* the values are BF16-representable */
                    }
                    if (!in) {
                        if ((k & 255u) == 255u && sm->abort_flag) break;
                        __nanosleep(64);
                    }
                }
                if (!in) { bad = true; continue; }
            }
            uint32_t *dst = (uint32_t *)(xs + (size_t)m * pl.K + (size_t)col * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) *(uint4 *)(dst + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                ss[m] = fmaf(bf16_lo(v[q]), bf16_lo(v[q]), ss[m]);
                ss[m] = fmaf(bf16_hi(v[q]), bf16_hi(v[q]), ss[m]);
            }
        }
    }
    if (__any_sync(0xffffffffu, bad)) { if (lane == 0) km_give_up(sm, P.status, ST_NEXT_X); return false; }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const float tot = warp_sum(ss[m]);
        if (lane == 0) sm->norm_red[m][wp] = tot;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->x_ready);
    return true;
}

/* ---- consumers: one layer ----------------------------------------------------------------------- */
template <int CIT, int MT>
__device__ __forceinline__ bool km_consumer_layer(const KmParams &P, KmSmem *sm, uint16_t *xs, uint8_t *ring, int l,
                                                  int kb0, int kb1, int ring_tile0, int part_tile0) {
    constexpr int NVROW = 2 * MT;
    constexpr int VALS = 4 * MT;      /* values a thread carries through a phase-1 tile */
    constexpr int JTM = VALS / NVROW; /* = 2 row steps per thread per tile */
    const PhasePlan &pl = P.p1;
    const KmLayer &LY = P.layers[l];
    const int stage_bytes = P.stage_bytes, nstages = P.nstages;
    const uint32_t ring_addr = smem_u32(ring);
    const int ti = threadIdx.x - 32, lane = threadIdx.x & 31;
    const bool active = ti < pl.CT * pl.RG;
    const int ct = ti % pl.CT, rg = ti / pl.CT;
    const unsigned hmask = 0xFFFFu << (lane & 16);
    const int G = (int)gridDim.x;
    const int pair0 = kb0 * 8, pair1 = kb1 * 8;
    const int nt1 = (pair1 - pair0 + pl.TR - 1) / pl.TR;
    const int nkb = kb1 - kb0;
    const int nt2 = (nkb + P.R2 - 1) / P.R2;

    /* ---------------- the layer's input: staged by the loader threads, prepared by everyone ------- */
    if (!km_stage_input<CIT, MT>(P, sm, xs, l)) return false;
    if (!mbar_wait<32>(&sm->x_ready, (uint32_t)l & 1u, &sm->abort_flag)) {
        km_give_up(sm, P.status, ST_NEXT_X);
        return false;
    }
    XChunk xc[CIT][MT];
    {
        float inv_rms[MT];
        const bool normalize = LY.norm_w != nullptr;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            inv_rms[m] = 1.0f;
            if (normalize) {
                float total = 0.0f;
                const int loader_warps = (pl.CT + 31) / 32;
                for (int w = 0; w < loader_warps; ++w) total += sm->norm_red[m][w];
                inv_rms[m] = rsqrtf(total / (float)pl.K + P.norm_eps);
            }
        }
#pragma unroll
        for (int c = 0; c < CIT; ++c)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int col = ct + c * pl.CT;
                const bool on = active && col < pl.cpr;
                uint32_t xv[16];
                load_chunk<false>(xv, xs + (size_t)m * pl.K + (size_t)min(col, pl.cpr - 1) * 32, on);
                prepare_chunk(xc[c][m], xv, on, normalize ? LY.norm_w + (size_t)min(col, pl.cpr - 1) * 32 : nullptr, inv_rms[m],
                              P.norm_gemma ? 1.0f : 0.0f);
            }
    }
    if (threadIdx.x == 32 && l == 0) km_stamp(P, 2);

    /* ---------------- phase 1: this CTA's gate/up row pairs --------------------------------------- */
    for (int lt = 0; lt < nt1; ++lt) {
        const int rt = ring_tile0 + lt, pt = part_tile0 + lt;
        const int s = rt % nstages;
        const int rows = min(pl.TR, pair1 - (pair0 + lt * pl.TR));
        if (!mbar_wait<32>(&sm->full[s], (uint32_t)(rt / nstages) & 1u, &sm->abort_flag)) {
            km_give_up(sm, P.status, ST_CONSUMER_FULL);
            return false;
        }
        if (threadIdx.x == 32 && lt == 0 && l == 0) km_stamp(P, 3);
        const int row0 = pair0 + lt * pl.TR;
        const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)stage_bytes;
        const uint32_t sc0 = st + (uint32_t)P.stage_w_bytes + (((uint32_t)row0 * (uint32_t)pl.G * 2u) & 15u);
        const uint32_t sc1 = st + (uint32_t)(P.stage_w_bytes + P.sc_half_bytes) +
                             (((uint32_t)(row0 + pl.up_offset) * (uint32_t)pl.G * 2u) & 15u);
        const int pslot = pt % kPartSlots;
        if (pt >= kPartSlots) { /* the epilogue must have drained this partial slot */
            if (!mbar_wait<100>(&sm->part_empty[pslot], (uint32_t)(pt / kPartSlots - 1) & 1u, &sm->abort_flag)) {
                km_give_up(sm, P.status, ST_PART_EMPTY);
                return false;
            }
        }
        float *part = sm->part + (size_t)pslot * (MT == 1 ? kPartFloats1 : kPartFloats2);
        float val[VALS];
#pragma unroll
        for (int v = 0; v < VALS; ++v) val[v] = 0.0f;
        if (active) {
            /* no data-dependent branches: a column chunk past the row end reads a clamped address
             * against an all-zero prepared slice, a row past the tile end reads the tile's last row
             * and its value is dropped at the store */
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
                    const uint32_t wp_ = st + (uint32_t)pj * (uint32_t)pl.rb;
                    const uint32_t s0p = sc0 + (uint32_t)pj * (uint32_t)pl.G * 2u, s1p = sc1 + (uint32_t)pj * (uint32_t)pl.G * 2u;
                    uint4 w0[CIT], w1[CIT];
                    float f0[CIT], f1[CIT];
#pragma unroll
                    for (int c = 0; c < CIT; ++c) {
                        w0[c] = lds16_at(wp_ + coff[c]);
                        f0[c] = lds_bf16_at(s0p + soff[c]);
                        w1[c] = lds16_at(wp_ + up_bytes + coff[c]);
                        f1[c] = lds_bf16_at(s1p + soff[c]);
                    }
#pragma unroll
                    for (int c = 0; c < CIT; ++c) {
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            val[j * NVROW + m] = fmaf((float)chunk_dot(w0[c], xc[c][m]), f0[c] * xc[c][m].fac, val[j * NVROW + m]);
                            val[j * NVROW + MT + m] = fmaf((float)chunk_dot(w1[c], xc[c][m]), f1[c] * xc[c][m].fac, val[j * NVROW + MT + m]);
                        }
                    }
                }
            }
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
    if (threadIdx.x == 32 && l == 0) km_stamp(P, 4);

    /* ---------------- phase 2: every output row against this CTA's own act values ----------------- */
    if (nkb > 0 && !mbar_wait<64>(&sm->act_ready, (uint32_t)l & 1u, &sm->abort_flag)) {
        km_give_up(sm, P.status, ST_ACT_READY);
        return false;
    }
    if (threadIdx.x == 32 && l == 0) km_stamp(P, 6);
    const int H = P.H;
    const int npairs = (H / 2 + kConsumerThreads - 1) / kConsumerThreads; /* <= kKmMaxPairs, checked on the host */
    if (nkb > 0) {
        /* (the launch's layer count and call number were read by the epilogue warp and are published
         * by its arrivals at act_ready / p_open) */
        const unsigned tag = km_tag(sm->epoch + (unsigned)l);
        int acc[MT][2 * kKmMaxPairs];
        float y[MT][2 * kKmMaxPairs];
        uint32_t sc[kKmMaxPairs];
        int hcol[kKmMaxPairs]; /* first of the two output rows of pair j, clamped into range */
#pragma unroll
        for (int j = 0; j < kKmMaxPairs; ++j) {
            hcol[j] = min(2 * ti + 2 * kConsumerThreads * j, H - 2);
#pragma unroll
            for (int m = 0; m < MT; ++m) { acc[m][2 * j] = acc[m][2 * j + 1] = 0; y[m][2 * j] = y[m][2 * j + 1] = 0.0f; }
        }
        int grp = kb0 / kKmGroupKb;
#pragma unroll
        for (int j = 0; j < kKmMaxPairs; ++j)
            sc[j] = j < npairs ? __ldg((const uint32_t *)(LY.st + (size_t)grp * H + hcol[j])) : 0u;
        for (int lt = 0; lt < nt2; ++lt) {
            const int rt = ring_tile0 + nt1 + lt;
            const int s = rt % nstages;
            if (!mbar_wait<32>(&sm->full[s], (uint32_t)(rt / nstages) & 1u, &sm->abort_flag)) {
                km_give_up(sm, P.status, ST_CONSUMER_FULL);
                return false;
            }
            if (threadIdx.x == 32 && lt == 0 && l == 0) km_stamp(P, 7);
            const int r0 = kb0 + lt * P.R2, rows = min(P.R2, kb1 - r0);
            const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)stage_bytes;
            for (int r = 0; r < rows; ++r) {
                const int kb = r0 + r;
                uint4 pln[MT];
#pragma unroll
                for (int m = 0; m < MT; ++m) pln[m] = *(const uint4 *)sm->planes[m][kb - kb0]; /* broadcast */
                const uint32_t rowaddr = st + (uint32_t)r * (uint32_t)H * 4u;
#pragma unroll
                for (int j = 0; j < kKmMaxPairs; ++j) {
                    if (j < npairs) { /* uniform over the CTA */
                        const uint2 w = km_lds8(rowaddr + (uint32_t)hcol[j] * 4u);
                        const uint32_t ws[2] = {w.x, w.y};
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const uint32_t o = ws[q] & 0xF0F0F0F0u, e = (ws[q] << 4) & 0xF0F0F0F0u;
#pragma unroll
                            for (int m = 0; m < MT; ++m) {
                                int hi = dp4a_ss(e, pln[m].x, 0);
                                hi = dp4a_ss(o, pln[m].y, hi);
                                int lo = dp4a_su(e, pln[m].z, 0);
                                lo = dp4a_su(o, pln[m].w, lo);
                                acc[m][2 * j + q] += hi * 256 + lo; /* 16 * sum code*X of this k-block; a group stays below 2^31 */
                            }
                        }
                    }
                }
                const bool last = kb == kb1 - 1;
                if ((kb % kKmGroupKb) == kKmGroupKb - 1 || last) { /* a scale group (or this CTA's part of it) ends */
                    const int seg = kb / kKmGroupKb - kb0 / kKmGroupKb;
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float fac = sm->fac[m][seg];
#pragma unroll
                        for (int j = 0; j < kKmMaxPairs; ++j) {
                            if (j < npairs) {
                                y[m][2 * j] = fmaf((float)acc[m][2 * j], bf16_lo(sc[j]) * fac, y[m][2 * j]);
                                y[m][2 * j + 1] = fmaf((float)acc[m][2 * j + 1], bf16_hi(sc[j]) * fac, y[m][2 * j + 1]);
                                acc[m][2 * j] = acc[m][2 * j + 1] = 0;
                            }
                        }
                    }
                    if (!last) {
                        ++grp;
#pragma unroll
                        for (int j = 0; j < kKmMaxPairs; ++j)
                            if (j < npairs) sc[j] = __ldg((const uint32_t *)(LY.st + (size_t)grp * H + hcol[j]));
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->empty[s]);
        }
        /* this CTA's share of every output row, as tagged words */
        unsigned long long *mine = P.partial + (size_t)blockIdx.x * km_partial_stride(MT, H);
#pragma unroll
        for (int j = 0; j < kKmMaxPairs; ++j) {
            if (j < npairs && 2 * ti + 2 * kConsumerThreads * j < H) {
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    km_store2(mine + (size_t)m * H + hcol[j], km_word(y[m][2 * j], tag), km_word(y[m][2 * j + 1], tag));
            }
        }
    }
    __syncwarp();
    if (lane == 0 && atomicAdd(&sm->arrive_p, 1u) % kConsumerWarps == kConsumerWarps - 1) km_arrive_counter(P.sync + 0); /* the CTA's last warp */
    if (threadIdx.x == 32 && l == 0) km_stamp(P, 8);

    /* ---------------- the rows this CTA owns: sum over CTAs, cross-rank exchange, output ----------- */
    /* Groups of eight lanes take one (row, token) item at a time.  Lane s adds the partial sums of the
     * CTAs s, s+8, ... in ascending order, a fixed three-step butterfly adds the eight lane sums (the
     * same bits in every lane), so the result does not depend on timing.  Under tensor parallelism
     * lane s then sends the rank's sum to ranks s (and s+8), waits for rank s's (and s+8's) word in
     * this rank's own buffer, and the values are added in rank order. */
    if (!mbar_wait<64>(&sm->p_open, (uint32_t)l & 1u, &sm->abort_flag)) {
        if (lane == 0) km_give_up(sm, P.status, ST_PARTIALS);
        return false;
    }
    if (threadIdx.x == 32 && l == 0) km_stamp(P, 10);
    const unsigned tag = km_tag(sm->epoch + (unsigned)l);
    const unsigned tp_seq0 = sm->seq0;
    const int b2 = km_begin(H, blockIdx.x, G), e2 = km_begin(H, blockIdx.x + 1, G);
    const int nitems = (e2 - b2) * MT;
    const int s8 = lane & 7, grp8 = ti >> 3;
    constexpr int kGroups = kConsumerThreads / 8;
    const unsigned gmask = 0xFFu << (lane & 24);
    const int KB = P.I / 8;
    const unsigned seq = tp_seq0 + (unsigned)l;
    /* bit i: CTA s8 + 8i exists and owns k-blocks (a CTA without any stores nothing).  With at least as
     * many k-blocks as CTAs every CTA owns some, and no division is needed to know it. */
    unsigned use_mask = 0;
    if (KB >= G) {
        for (int i = 0; i < kKmMaxQ; ++i)
            if (s8 + 8 * i < G) use_mask |= 1u << i;
    } else {
        for (int i = 0; i < kKmMaxQ; ++i) {
            const int q = s8 + 8 * i;
            if (q < G && km_begin(KB, q + 1, G) > km_begin(KB, q, G)) use_mask |= 1u << i;
        }
    }
    bool failed = false;
    for (int it0 = 0; it0 < nitems; it0 += kGroups) { /* uniform trip count over the CTA */
        const int item = it0 + grp8;
        const bool valid = item < nitems;
        const int ic = valid ? item : 0;
        const int row = b2 + ic / MT, m = ic % MT;
        /* the words of this lane: all loads first, then the tag checks, so the loads overlap */
        unsigned long long w[kKmMaxQ];
        bool in = false;
        uint32_t attempts = 0;
        if (threadIdx.x == 32 && l == 0 && it0 == 0) km_stamp(P, 15);
        for (uint32_t k = 0; k < kTpPollLimit && !in; ++k) {
            in = true;
            ++attempts;
#pragma unroll
            for (int i = 0; i < kKmMaxQ; ++i) {
                w[i] = (unsigned long long)tag << 32; /* value 0.0, tag of this layer */
                if ((use_mask >> i) & 1u) w[i] = km_load1(P.partial + (size_t)(s8 + 8 * i) * km_partial_stride(MT, H) + (size_t)m * H + row);
            }
#pragma unroll
            for (int i = 0; i < kKmMaxQ; ++i) in = in && (unsigned)(w[i] >> 32) == tag;
            if (!in) {
                if ((k & 255u) == 255u && sm->abort_flag) break;
                __nanosleep(32);
            }
        }
        if (threadIdx.x == 32 && l == 0 && it0 == 0) { km_stamp(P, 11); if (P.trace) P.trace[(size_t)blockIdx.x * 16 + 14] = (long long)attempts; }
        float a = 0.0f;
#pragma unroll
        for (int i = 0; i < kKmMaxQ; ++i) a += __uint_as_float((unsigned)w[i]);
        const bool partials_missing = __any_sync(gmask, !in);
        bool bad = partials_missing;
        a += __shfl_xor_sync(gmask, a, 1);
        a += __shfl_xor_sync(gmask, a, 2);
        a += __shfl_xor_sync(gmask, a, 4);
        if (P.tp > 1) {
            const size_t elem = (size_t)m * H + row;
            const size_t off = (size_t)((seq & 1u) * P.tp + P.rank) * P.slot_stride + elem;
            if (valid && !bad)
                for (int r = s8; r < P.tp; r += 8) tp_store_tagged(P.peer_slots[r] + off, a, tp_tag(seq));
            const unsigned long long *mine = P.peer_slots[P.rank] + (size_t)(seq & 1u) * P.tp * P.slot_stride + elem;
            float v[2] = {0.0f, 0.0f};
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r = s8 + 8 * u;
                if (r < P.tp && valid && !bad) {
                    const unsigned long long *p = mine + (size_t)r * P.slot_stride;
                    bool got = tp_load_tagged(p, tp_tag(seq), &v[u]);
                    for (uint32_t k = 0; !got && k < kTpPollLimit; ++k) {
                        if ((k & 1023u) == 1023u && sm->abort_flag) break;
                        __nanosleep(20);
                        got = tp_load_tagged(p, tp_tag(seq), &v[u]);
                    }
                    if (!got) bad = true;
                }
            }
            float tot = 0.0f;
            for (int r = 0; r < P.tp; ++r) tot += __shfl_sync(gmask, r < 8 ? v[0] : v[1], (lane & 24) | (r & 7));
            a = tot;
        }
        bad = __any_sync(gmask, bad);
        if (bad) {
            if (valid && s8 == 0) km_give_up(sm, P.status, partials_missing ? ST_PARTIALS : ST_PEER_DATA);
            failed = true;
        } else if (valid && s8 == 0) {
            const size_t o = (size_t)m * H + row;
            const float yv = round_bf16(a);
            P.out[o] = f32_to_bf16_bits(yv);
            if (P.residual) {
                const float hold = bf16_bits_to_f32(P.residual_is_x ? xs[o] : P.residual[o]);
                const float hnew = round_bf16(hold + yv);
                P.residual[o] = f32_to_bf16_bits(hnew);
                if (l + 1 < P.L) km_store1(P.hx + o, km_word(hnew, tag));
            }
        }
    }
    __syncwarp();
    if (lane == 0 && atomicAdd(&sm->arrive_h, 1u) % kConsumerWarps == kConsumerWarps - 1) km_arrive_counter(P.sync + 1);
    if (threadIdx.x == 32 && l == 0) km_stamp(P, 9);
    return !failed;
}

/* ---- the kernel --------------------------------------------------------------------------------- */
template <int CIT, int MT>
__global__ void __launch_bounds__(kThreads, 1) ffn_kmajor_kernel(const __grid_constant__ KmParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    KmSmem *sm = (KmSmem *)smem_raw;
    uint16_t *xs = (uint16_t *)(smem_raw + km_smem_header(MT));
    uint8_t *ring = (uint8_t *)xs + P.xs_bytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0) {
        if (lane == 0) km_stamp(P, 0);
        if (lane < P.nstages) { mbar_init(&sm->full[lane], 1); mbar_init(&sm->empty[lane], kConsumerWarps); }
        if (lane >= 8 && lane < 8 + kPartSlots) { mbar_init(&sm->part_full[lane - 8], kConsumerWarps); mbar_init(&sm->part_empty[lane - 8], 1); }
        if (lane == 16) mbar_init(&sm->x_ready, (P.p1.CT + 31) / 32);
        if (lane == 17) mbar_init(&sm->act_ready, 1);
        if (lane == 18) mbar_init(&sm->p_open, 1);
        if (lane == 19) mbar_init(&sm->h_open, 1);
        if (lane == 20) { sm->arrive_p = 0; sm->arrive_h = 0; }
        if (lane == 31) sm->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
        /* the barriers exist: this warp (the producer) goes on at once, the others wait for it here */
        asm volatile("bar.arrive 1, %0;" ::"n"(kThreads) : "memory");
    } else {
        uint32_t pre[CIT][MT][16];
        km_prefetch_input<CIT, MT>(P, pre); /* in flight while warp 0 sets the barriers up */
        asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
        km_stage_first<CIT, MT>(P, sm, xs, pre);
    }
    const int G = (int)gridDim.x, KB = P.I / 8;
    const int kb0 = km_begin(KB, blockIdx.x, G), kb1 = km_begin(KB, blockIdx.x + 1, G);
    const int nt1 = ((kb1 - kb0) * 8 + P.p1.TR - 1) / P.p1.TR;
    const int nt2 = (kb1 - kb0 + P.R2 - 1) / P.R2;

    if (warp == 0) {
        if (lane == 0) {
            km_stamp(P, 1);
            km_producer(P, sm, ring, kb0, kb1);
        }
    } else if (warp <= kConsumerWarps) {
        for (int l = 0; l < P.L; ++l)
            if (!km_consumer_layer<CIT, MT>(P, sm, xs, ring, l, kb0, kb1, l * (nt1 + nt2), l * nt1)) break;
    } else {
        unsigned base = 0;
        for (int l = 0; l < P.L; ++l)
            if (!km_epilogue_layer<MT>(P, sm, l, kb0, kb1, l * nt1, base)) break;
    }
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0 && !sm->abort_flag) {
        P.sync[2] = sm->base + (unsigned)P.L * (unsigned)G;
        P.sync[3] = sm->epoch + (unsigned)P.L;
        if (P.tp > 1) atomicAdd(P.tp_seq, (unsigned)P.L);
        km_stamp(P, 12);
    }
}

/* word-level transpose of the packed down projection: w [H][KB] -> wt [KB][H] (32-bit words) */
__global__ void km_transpose_words_kernel(uint32_t *__restrict__ wt, const uint32_t *__restrict__ w, int H, int KB) {
    __shared__ uint32_t tile[32][33];
    const int kb0 = blockIdx.x * 32, h0 = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y)
        if (h0 + r < H && kb0 + (int)threadIdx.x < KB) tile[r][threadIdx.x] = w[(size_t)(h0 + r) * KB + kb0 + threadIdx.x];
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y)
        if (kb0 + r < KB && h0 + (int)threadIdx.x < H) wt[(size_t)(kb0 + r) * H + h0 + threadIdx.x] = tile[threadIdx.x][r];
}
/* scales [H][G] -> [G][H] */
__global__ void km_transpose_scales_kernel(uint16_t *__restrict__ st, const uint16_t *__restrict__ s, int H, int G) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; /* index into st */
    if (i >= (size_t)H * G) return;
    const int g = (int)(i / H), h = (int)(i % H);
    st[i] = s[(size_t)h * G + g];
}

/* ============================================================================================= */
/* Host side                                                                                     */
/* ============================================================================================= */
constexpr int kKmBufTokens = 4; /* tokens the hand-over buffers are sized for (the tensor-core kernel takes up to four) */
struct KmDevice {
    bool ready = false;
    int sm_count = 0, smem_optin = 0, cooperative = 0;
    unsigned *sync = nullptr;              /* 4 words */
    unsigned long long *partial = nullptr; /* [sm_count][kKmBufTokens][hidden_cap] */
    unsigned long long *hx = nullptr;      /* [kKmBufTokens][hidden_cap] */
    int hidden_cap = 0;
    bool attr_set[2][2] = {};
};
static KmDevice g_km[64];
static std::mutex g_km_mutex;

/* The k-major copies, by the device address of the row-major down projection they were made from. */
struct KmPrepared {
    uint32_t *wt = nullptr;
    uint16_t *st = nullptr;
    int hidden = 0, inter = 0, device = 0;
};
static std::unordered_map<const void *, KmPrepared> g_km_layers;

static int km_device(KmDevice **out, int hidden) {
    int dev = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FFN_ERR_CONFIG, "device index %d out of range", dev);
    KmDevice &d = g_km[dev];
    if (!d.ready) {
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev), "SM count");
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "smem opt-in");
        FFN_CUDA_TRY(cudaDeviceGetAttribute(&d.cooperative, cudaDevAttrCooperativeLaunch, dev), "cooperative launch");
        if (cudaMalloc(&d.sync, 4 * sizeof(unsigned)) != cudaSuccess)
            return fail(FFN_ERR_ALLOC, "cannot allocate the k-major kernel's synchronisation words");
        FFN_CUDA_TRY(cudaMemset(d.sync, 0, 4 * sizeof(unsigned)), "clear synchronisation words");
        d.ready = true;
    }
    if (hidden > d.hidden_cap) { /* first use of a wider model on this device: (re)allocate the hand-over buffers */
        if (d.partial) { FFN_CUDA_TRY(cudaDeviceSynchronize(), "k-major kernel: scratch regrow"); cudaFree(d.partial); cudaFree(d.hx); }
        d.partial = nullptr; d.hx = nullptr; d.hidden_cap = 0;
        const size_t pw = (size_t)d.sm_count * km_partial_stride(kKmBufTokens, hidden), hw = (size_t)kKmBufTokens * hidden;
        if (cudaMalloc(&d.partial, pw * 8) != cudaSuccess || cudaMalloc(&d.hx, hw * 8) != cudaSuccess) {
            (void)cudaGetLastError();
            if (d.partial) cudaFree(d.partial);
            d.partial = nullptr;
            return fail(FFN_ERR_ALLOC, "k-major kernel: cannot allocate %zu bytes of hand-over buffers", (pw + hw) * 8);
        }
        /* tag 0 marks a word nobody has written */
        FFN_CUDA_TRY(cudaMemset(d.partial, 0, pw * 8), "clear hand-over buffers");
        FFN_CUDA_TRY(cudaMemset(d.hx, 0, hw * 8), "clear hand-over buffers");
        d.hidden_cap = hidden;
    }
    *out = &d;
    return FFN_OK;
}

int kmajor_device_view(int hidden, int tokens, KmDeviceView *out) {
    if (tokens > kKmBufTokens) return fail(FFN_ERR_CONFIG, "k-major kernels: at most %d tokens", kKmBufTokens);
    std::lock_guard<std::mutex> lock(g_km_mutex);
    KmDevice *d = nullptr;
    const int st = km_device(&d, hidden);
    if (st) return st;
    out->sm_count = d->sm_count; out->smem_optin = d->smem_optin; out->cooperative = d->cooperative;
    out->sync = d->sync; out->partial = d->partial; out->hx = d->hx;
    return FFN_OK;
}

bool kmajor_lookup(const void *down_i4, int hidden, int inter, int dev, const uint32_t **wt, const uint16_t **st) {
    std::lock_guard<std::mutex> lock(g_km_mutex);
    const auto it = g_km_layers.find(down_i4);
    if (it == g_km_layers.end() || it->second.hidden != hidden || it->second.inter != inter || it->second.device != dev) return false;
    *wt = it->second.wt;
    *st = it->second.st;
    return true;
}

/* Clears the kernel's counters after a launch that gave up (called when the status word is reset). */
void kmajor_reset_sync() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    std::lock_guard<std::mutex> lock(g_km_mutex);
    KmDevice &d = g_km[dev];
    if (!d.ready) return;
    (void)cudaMemset(d.sync, 0, 4 * sizeof(unsigned));
    /* the layer count (the tags' base) starts again at zero, so no word of the interrupted launches may survive */
    if (d.partial) (void)cudaMemset(d.partial, 0, (size_t)d.sm_count * km_partial_stride(kKmBufTokens, d.hidden_cap) * 8);
    if (d.hx) (void)cudaMemset(d.hx, 0, (size_t)kKmBufTokens * d.hidden_cap * 8);
}

/* Launch geometry from the shape alone.  Returns false when the kernel does not take it. */
static bool km_plan(KmParams &P, int tokens, int H, int I, int grid, int smem_optin, int &c1, size_t &smem) {
    if (tokens < 1 || tokens > 2) return false;
    if (H <= 0 || I <= 0 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP) return false;
    if (H > 2 * kConsumerThreads * kKmMaxPairs || I > (1 << 22)) return false;
    if (grid < 1 || grid > 8 * kKmMaxQ) return false;
    const int KB = I / 8;
    if ((KB + grid - 1) / grid > kKmMaxKb) return false;
    P.M = tokens; P.H = H; P.I = I;
    if (!plan_phase(P.p1, H, tokens, true, kDefaultStageTarget, c1)) return false;
    P.p1.rows_total = I; P.p1.up_offset = I;
    const int part_floats = tokens == 1 ? kPartFloats1 : kPartFloats2;
    if (P.p1.TR * 2 * tokens * P.p1.nhw > part_floats) return false;
    P.stage_w_bytes = round_up(2 * P.p1.TR * P.p1.rb, 128);
    P.R2 = max(1, min(kKmMaxKb, P.stage_w_bytes / (H * 4))); /* k-major rows per stage: about what a gate/up tile takes */
    P.sc_half_bytes = round_up(P.p1.TR * P.p1.G * 2 + 32, 16);
    P.stage_bytes = round_up(max(P.stage_w_bytes + 2 * P.sc_half_bytes, P.R2 * H * 4), 128);
    P.xs_bytes = round_up(tokens * H * 2, 128);
    const size_t fixed = km_smem_header(tokens) + (size_t)P.xs_bytes;
    if (fixed + 2 * (size_t)P.stage_bytes > (size_t)smem_optin) return false;
    P.nstages = (int)min((size_t)kMaxStages, ((size_t)smem_optin - fixed) / (size_t)P.stage_bytes);
    smem = fixed + (size_t)P.nstages * P.stage_bytes;
    return true;
}

bool kmajor_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes) {
    static KmParams P; /* large: not on the stack */
    std::lock_guard<std::mutex> lock(g_km_mutex);
    P = KmParams();
    int c1 = 0;
    size_t smem = 0;
    if (!km_plan(P, tokens, H, I, sm_count, smem_optin, c1, smem)) return false;
    const int KB = I / 8;
    snprintf(out, out_bytes,
             "kernel=kmajor grid=%d threads=%d smem=%zu stages=%d stage_bytes=%d x_bytes=%d p1_cit=%d p1_ct=%d p1_rg=%d p1_jt=%d "
             "p1_pairs_per_tile=%d p2_kmajor_rows_per_tile=%d kblocks_per_cta=%d..%d column_pairs_per_thread=%d",
             sm_count, kThreads, smem, P.nstages, P.stage_bytes, P.xs_bytes, c1, P.p1.CT, P.p1.RG, P.p1.JT, P.p1.TR, P.R2,
             KB / sm_count, (KB + sm_count - 1) / sm_count, (H / 2 + kConsumerThreads - 1) / kConsumerThreads);
    return true;
}

template <int C1, int MT>
static int km_launch(KmDevice &d, const KmParams &P, int grid, size_t smem, cudaStream_t stream) {
    bool &set = d.attr_set[C1 - 1][MT - 1];
    if (!set) {
        FFN_CUDA_TRY(cudaFuncSetAttribute(ffn_kmajor_kernel<C1, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, d.smem_optin),
                     "k-major FFN: shared-memory opt-in");
        set = true;
    }
    void *args[] = {(void *)&P};
    FFN_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)ffn_kmajor_kernel<C1, MT>, dim3(grid), dim3(kThreads), args, smem, stream),
                 "k-major FFN launch");
    return FFN_OK;
}

static_assert(sizeof(KmParams) <= 4000, "the kernel parameters must fit the 4 KB parameter space");

/* `num_layers` layers (1 for a single FFN call) in launches of at most kKmMaxLayers.  Returns
 * FFN_NOT_ADMITTED when a layer has no k-major copy or the shape is outside what the kernel takes;
 * nothing has been launched then. */
static int g_prefer_dp4a = 1; /* measured: the dp4a kernel is the faster and the more precise of the two */
int kmajor_prefer_dp4a(int on) {
    const int old = g_prefer_dp4a;
    g_prefer_dp4a = on != 0;
    return old;
}

int kmajor_ffn_launch(cudaStream_t stream, const void *x, void *act, void *layer_out, const FfnMlpWeights *layers,
                      int num_layers, int tokens, int H, int I, const FusedTp *tp, void *residual, int with_norm,
                      float eps, int gemma, unsigned *status) {
    if (!g_prefer_dp4a) { /* the tensor-core consumers first; shapes they do not take fall through to the dp4a kernel */
        const int st = imma_ffn_launch(stream, x, act, layer_out, layers, num_layers, tokens, H, I, tp, residual, with_norm, eps,
                                       gemma, status);
        if (st != FFN_NOT_ADMITTED) return st;
    }
    if (tokens < 1 || tokens > 2 || num_layers < 1) return FFN_NOT_ADMITTED;
    if (num_layers > 1 && (residual != x || !with_norm)) return FFN_NOT_ADMITTED; /* a stack runs on the residual stream */
    std::lock_guard<std::mutex> lock(g_km_mutex);
    int dev = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    for (int l = 0; l < num_layers; ++l) {
        const auto it = g_km_layers.find(layers[l].down_i4);
        if (it == g_km_layers.end() || it->second.hidden != H || it->second.inter != I || it->second.device != dev) return FFN_NOT_ADMITTED;
        if (((uintptr_t)layers[l].gate_up_i4 & 15) || ((uintptr_t)layers[l].gate_up_i4_scales & 15)) return FFN_NOT_ADMITTED;
        if (with_norm && (!layers[l].post_norm_w || ((uintptr_t)layers[l].post_norm_w & 15))) return FFN_NOT_ADMITTED;
    }
    if (((uintptr_t)x & 15) || ((uintptr_t)act & 1)) return FFN_NOT_ADMITTED;
    KmDevice *dp = nullptr;
    const int st = km_device(&dp, H);
    if (st) return st;
    KmDevice &d = *dp;
    if (!d.cooperative) return FFN_NOT_ADMITTED;
    static KmParams P; /* 3 KB; guarded by the mutex above */
    P = KmParams();
    int c1 = 0;
    size_t smem = 0;
    const int grid = d.sm_count; /* under TP every rank runs the same grid: CTA c owns the same rows everywhere */
    if (!km_plan(P, tokens, H, I, grid, d.smem_optin, c1, smem)) return FFN_NOT_ADMITTED;
    P.x = (const uint16_t *)x;
    P.act = (uint16_t *)act;
    P.out = (uint16_t *)layer_out;
    P.residual = (uint16_t *)residual;
    P.residual_is_x = residual != nullptr && residual == x;
    P.sync = d.sync;
    P.status = status;
    P.partial = d.partial;
    P.hx = d.hx;
    P.tp = 1; P.rank = 0;
    if (tp && tp->tp > 1) {
        P.tp = tp->tp; P.rank = tp->rank; P.peer_slots = tp->peer_slots; P.slot_stride = tp->slot_stride; P.tp_seq = tp->seq;
        if (tokens * H > tp->slot_stride) return fail(FFN_ERR_CONFIG, "k-major FFN: %d tokens exceed the exchange buffer", tokens);
    }
    P.norm_eps = eps; P.norm_gemma = gemma;
    P.trace = fused_get_trace();
    for (int l0 = 0; l0 < num_layers; l0 += kKmMaxLayers) {
        P.L = min(kKmMaxLayers, num_layers - l0);
        for (int l = 0; l < P.L; ++l) {
            const FfnMlpWeights &w = layers[l0 + l];
            const KmPrepared &pr = g_km_layers[w.down_i4];
            P.layers[l] = {w.gate_up_i4, (const uint16_t *)w.gate_up_i4_scales, pr.wt, pr.st,
                           with_norm ? (const uint16_t *)w.post_norm_w : nullptr};
        }
        int rc;
        if (tokens == 2) rc = km_launch<1, 2>(d, P, grid, smem, stream);
        else if (c1 == 1) rc = km_launch<1, 1>(d, P, grid, smem, stream);
        else rc = km_launch<2, 1>(d, P, grid, smem, stream);
        if (rc) return rc;
    }
    return FFN_OK;
}

}  // namespace ffn

using namespace ffn;

extern "C" {

int ffn_decode_layer_prepare(const FfnMlpWeights *w, const FfnModelDims *dims, void *stream) {
    clear_error();
    if (!w || !dims) return fail(FFN_ERR_CONFIG, "ffn_decode_layer_prepare: null weights or dims");
    if (!w->down_i4 || !w->down_i4_scales) return fail(FFN_ERR_CONFIG, "ffn_decode_layer_prepare: the layer carries no INT4 down projection");
    if (w->i4_group != FFN_INT4_GROUP) return fail(FFN_ERR_CONFIG, "ffn_decode_layer_prepare: this format's group is %d, not %d", FFN_INT4_GROUP, w->i4_group);
    const int H = dims->hidden_size, I = dims->intermediate_size;
    if (H <= 0 || I <= 0 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "ffn_decode_layer_prepare: hidden=%d / intermediate=%d are not whole numbers of %d-wide groups", H, I, FFN_INT4_GROUP);
    if (((uintptr_t)w->down_i4 & 3) || ((uintptr_t)w->down_i4_scales & 1)) return fail(FFN_ERR_CONFIG, "ffn_decode_layer_prepare: misaligned operand");
    int dev = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    std::lock_guard<std::mutex> lock(g_km_mutex);
    KmPrepared &pr = g_km_layers[w->down_i4];
    const int KB = I / 8, G = I / FFN_INT4_GROUP;
    if (pr.wt && (pr.hidden != H || pr.inter != I || pr.device != dev)) { /* the address now holds another matrix */
        cudaFree(pr.wt); cudaFree(pr.st);
        pr = KmPrepared();
    }
    if (!pr.wt) {
        if (cudaMalloc(&pr.wt, (size_t)KB * H * 4) != cudaSuccess || cudaMalloc(&pr.st, (size_t)G * H * 2) != cudaSuccess) {
            (void)cudaGetLastError();
            if (pr.wt) cudaFree(pr.wt);
            g_km_layers.erase(w->down_i4);
            return fail(FFN_ERR_ALLOC, "ffn_decode_layer_prepare: cannot allocate the k-major copy (%zu bytes)", (size_t)KB * H * 4 + (size_t)G * H * 2);
        }
        pr.hidden = H; pr.inter = I; pr.device = dev;
    }
    cudaStream_t s = (cudaStream_t)stream;
    km_transpose_words_kernel<<<dim3((KB + 31) / 32, (H + 31) / 32), dim3(32, 8), 0, s>>>(pr.wt, (const uint32_t *)w->down_i4, H, KB);
    FFN_CUDA_TRY(cudaGetLastError(), "ffn_decode_layer_prepare: transpose launch");
    const size_t n = (size_t)H * G;
    km_transpose_scales_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(pr.st, (const uint16_t *)w->down_i4_scales, H, G);
    FFN_CUDA_TRY(cudaGetLastError(), "ffn_decode_layer_prepare: transpose launch");
    return FFN_OK;
}

int ffn_decode_layer_release(const FfnMlpWeights *w) {
    clear_error();
    if (!w || !w->down_i4) return FFN_OK;
    std::lock_guard<std::mutex> lock(g_km_mutex);
    const auto it = g_km_layers.find(w->down_i4);
    if (it == g_km_layers.end()) return FFN_OK;
    int restore = 0;
    (void)cudaGetDevice(&restore);
    (void)cudaSetDevice(it->second.device);
    (void)cudaDeviceSynchronize();
    cudaFree(it->second.wt);
    cudaFree(it->second.st);
    (void)cudaSetDevice(restore);
    (void)cudaGetLastError();
    g_km_layers.erase(it);
    return FFN_OK;
}

int ffn_decode_layer_is_prepared(const FfnMlpWeights *w) {
    if (!w || !w->down_i4) return 0;
    std::lock_guard<std::mutex> lock(g_km_mutex);
    return g_km_layers.count(w->down_i4) ? 1 : 0;
}

}  // extern "C"
