/*
 * ffn_imma.cu - the decode-shaped INT4 FFN (1..4 tokens), one or many layers, as ONE persistent kernel
 * whose inner products run on the INT8 tensor cores.
 *
 * Structure and hand-over protocol are those of ffn_kmajor.cu (k-major copy of the down projection,
 * every CTA multiplies the down projection against the act values it produced itself, partial sums and
 * the residual stream travel as tagged words).  What changes is the consumers' arithmetic.  OPT-IN
 * (ffn_int4_set_decode_kernel(0)): on B200 this variant measured slower than the dp4a kernels (54.7 us
 * against 40.6 / 30.3 us per 5120 x 17408 layer - the legacy mma.sync integer path is slow there) and its
 * 15-bit planes with one exponent per 128 values are coarser than their 16 bits per 32.  The idea: with
 * dp4a a thread spends 7..10 instructions per 8 codes, and 17 warps of such work keep pace with the
 * HBM stream only barely: every stall of the pipeline is lost time.  Here a 4-bit code is still
 * widened to the signed byte 16*code with one logic operation per four codes, but the products are
 * formed by mma.sync.m16n8k32 (s8 x s8 -> s32): 16 weight rows x 32 codes per instruction against the
 * activations as two signed byte planes per token (15-bit block fixed point: X = hi*256 + lo, both in
 * [-128, 127]; one exponent per 128-group, so a group accumulates in INT32 inside the tensor core and
 * is scaled once in FP32 - exact integer arithmetic inside a group, like the dp4a kernels).  The eight
 * MMA columns hold {hi, lo} of up to four tokens, so two, three or four tokens cost what one does.
 *
 *   phase 1  a tile is one k-block of act: 8 gate rows + 8 up rows over all of K, i.e. exactly one
 *            16-row MMA tile; rows sit in shared memory with a 16-byte skew so that the A-fragment
 *            loads are bank-conflict free.  Warp w takes the 128-groups [w*gpp, (w+1)*gpp) of the tile;
 *            thread (g, t) ends with the gate and the up sum of pair g for token t.  The epilogue warp
 *            adds the warps' partial sums in warp order, rounds, applies SiLU*up.
 *   phase 2  a tile is one chunk (<= 4 k-blocks of one 128-group) of one slab of output rows; warp w
 *            takes the 16-row blocks w, w+17, ... of the slab.  INT32 accumulators persist over the
 *            chunks of a group, FP32 sums over the groups; at the end of a slab they leave as tagged
 *            words.
 */
#include <stdio.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "stream_common.cuh"
#include "kmajor_common.cuh"

namespace ffn {

constexpr int kImMaxLayers = 64;
constexpr int kImMaxTokens = 4;
constexpr int kImMaxKb = 16;          /* k-blocks one CTA may own: its K range touches at most two 128-groups */
constexpr int kImMaxSeg = 2;
constexpr int kImMaxChunks = 6;       /* chunks of <= 4 k-blocks that never cross a group boundary */
constexpr int kImMaxParts = 16;       /* K parts of a phase-1 tile, one per warp */
constexpr int kImMaxRb = 5;           /* 16-row blocks of a slab one warp takes: slab <= 17 * 5 * 16 rows */
constexpr int kImMaxQ = 20;           /* partial sums one reducer lane adds: grid <= 8 * 20 */
constexpr int kImMaxGroups = 64;      /* 128-groups of the hidden size */
constexpr int kImGroupKb = FFN_INT4_GROUP / 8;

struct ImLayer {
    const uint8_t *gu_w;
    const uint16_t *gu_s;
    const uint32_t *wt;
    const uint16_t *st;
    const uint16_t *norm_w;
};

struct ImParams {
    const uint16_t *x;
    uint16_t *act;
    uint16_t *out;
    uint16_t *residual;
    int residual_is_x;
    int M, H, I, L;
    int G1;                   /* 128-groups of the hidden size */
    int rb1, rs1;             /* gate/up row bytes (H/2) and their stride in a stage (rb1 + 16) */
    int nparts, gpp;          /* K parts of a phase-1 tile and groups per part */
    int slab, nslabs, rs2;    /* output rows per phase-2 slab, slabs, row stride of a chunk row in a stage (slab*4 + 32) */
    int stage_bytes, nstages, sc_off, sc_half_bytes;
    int xp_bytes, xs_bytes;   /* activation byte planes, raw activations (both [M][H]-sized) */
    unsigned *sync;
    unsigned *status;
    unsigned long long *partial;
    unsigned long long *hx;
    int tp, rank, slot_stride;
    unsigned long long *const *peer_slots;
    unsigned *tp_seq;
    float norm_eps;
    int norm_gemma;
    long long *trace;
    ImLayer layers[kImMaxLayers];
};

struct ImSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t part_full[kPartSlots];
    uint64_t part_empty[kPartSlots];
    uint64_t x_ready;         /* raw input of the layer staged (loader warps arrive) */
    uint64_t xp_ready;        /* its byte planes built (every consumer warp arrives) */
    uint64_t act_ready;       /* this CTA's act values and their byte planes (epilogue arrives) */
    uint64_t st_full;         /* the down projection's scale rows of this CTA's groups (bulk copies) */
    uint64_t p_open;
    uint64_t h_open;
    unsigned arrive_p, arrive_h;
    int abort_flag;
    unsigned base, epoch, seq0;
    int nchunks, nseg;
    int chunk_kb[kImMaxChunks];   /* first k-block (absolute) */
    int chunk_n[kImMaxChunks];    /* k-blocks in the chunk, 1..4 */
    int chunk_seg[kImMaxChunks];  /* which of this CTA's group segments */
    float norm_red[kImMaxTokens][kConsumerWarps + 3];
    float xfac[kImMaxTokens][kImMaxGroups];
    float afac[kImMaxTokens][kImMaxSeg + 2];
    __align__(16) uint32_t planes[kImMaxTokens][kImMaxKb][4]; /* [token][k-block]{hi even, hi odd, lo even, lo odd} */
    uint16_t act_s[kImMaxTokens][kImMaxKb * 8];
    float part[1];            /* kPartSlots slots of 8 pairs x 2 x tokens x nparts floats follow */
};

__host__ __device__ constexpr int im_part_floats(int tokens) { return 8 * 2 * tokens * kImMaxParts; }
__host__ __device__ constexpr size_t im_smem_header(int tokens) {
    return (sizeof(ImSmem) + (size_t)kPartSlots * im_part_floats(tokens) * sizeof(float) + 127) / 128 * 128;
}

__device__ __forceinline__ void im_give_up(ImSmem *sm, unsigned *status, int where) {
    sm->abort_flag = 1;
    atomicCAS(status, 0u, (unsigned)where | ((unsigned)blockIdx.x << 8));
}
__device__ __forceinline__ void im_stamp(const ImParams &P, int slot) {
    if (P.trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        P.trace[(size_t)blockIdx.x * 16 + slot] = (long long)t;
    }
}
__device__ __forceinline__ uint32_t im_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
/* D (16x8, s32) += A (16x32, s8, row) * B (32x8, s8, col).  Lane (g = lane / 4, t = lane % 4) holds
 * a0: row g, k 4t..4t+3; a1: row g+8, same k; a2: row g, k 16+4t..; a3: row g+8, k 16+4t..;
 * b0: k 4t..4t+3 of column g; b1: k 16+4t.. of column g; d0, d1: row g, columns 2t, 2t+1; d2, d3: row g+8. */
__device__ __forceinline__ void im_mma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/* 15-bit block fixed point of eight activations, as the four byte planes of one weight word:
 * X = rint(x * 2^(13-E)) in [-16320, 16320], X = hi * 256 + lo with lo the SIGNED low byte, so that
 * both planes are signed bytes (|hi| <= 64).  Plane byte i pairs with code 2i (even planes) or 2i+1
 * (odd planes) of the word.  Returns {hi even, hi odd, lo even, lo odd}. */
__device__ __forceinline__ uint4 im_planes(const float (&v)[8], float up) {
    uint32_t hi_e = 0, hi_o = 0, lo_e = 0, lo_o = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        /* 1.5*2^23 + v*up has the rounded (nearest-even) integer in its low mantissa bits */
        const int X = (int)(short)(__float_as_int(fmaf(v[i], up, 12582912.0f)) & 0xFFFF);
        const int lo = (int)(signed char)(X & 0xFF);
        const int hi = (X - lo) >> 8;
        const uint32_t sh = 8u * (uint32_t)(i >> 1);
        if (i & 1) { hi_o |= ((uint32_t)hi & 0xFFu) << sh; lo_o |= ((uint32_t)lo & 0xFFu) << sh; }
        else       { hi_e |= ((uint32_t)hi & 0xFFu) << sh; lo_e |= ((uint32_t)lo & 0xFFu) << sh; }
    }
    return make_uint4(hi_e, hi_o, lo_e, lo_o);
}
/* exponent field E of the largest magnitude -> the scaling of X and the factor that undoes it together
 * with the 16 the widened codes carry.  E < 19 counts as an all-zero block; a block with an Inf or a
 * NaN (E == 255) gets fac = NaN, so that non-finite inputs give non-finite outputs. */
__device__ __forceinline__ void im_scaling(int E, float &up, float &fac) {
    const bool live = E >= 19 && E < 255;
    up = live ? __uint_as_float((uint32_t)(267 - E) << 23) : 0.0f;                 /* 2^(140-E) */
    fac = live ? __uint_as_float((uint32_t)(E - 17) << 23)                         /* 2^(E-140) / 16 */
               : (E == 255 ? __uint_as_float(0x7FC00000u) : 0.0f);
}

/* ---- this CTA's phase-2 chunks ------------------------------------------------------------------- */
/* The K range [kb0, kb1) in chunks of at most four k-blocks that do not cross a 128-group boundary
 * (one MMA covers four k-blocks and a group's INT32 sums must not mix with the next group's). */
__device__ __forceinline__ int im_build_chunks(int kb0, int kb1, int *ckb, int *cn, int *cseg, int *nseg_out) {
    int n = 0, nseg = 0;
    for (int g = kb0 / kImGroupKb; g * kImGroupKb < kb1 && kb1 > kb0; ++g, ++nseg) {
        const int lo = max(kb0, g * kImGroupKb), hi = min(kb1, (g + 1) * kImGroupKb);
        for (int kb = lo; kb < hi && n < kImMaxChunks; kb += 4, ++n) {
            ckb[n] = kb; cn[n] = min(4, hi - kb); cseg[n] = nseg;
        }
    }
    *nseg_out = nseg;
    return n;
}

/* ---- producer: the weight stream of all layers ---------------------------------------------------- */
/* Phase-1 tile lt: the 8 gate rows and the 8 up rows of pairs [8(kb0+lt), +8), each row its own bulk
 * copy (the rows are skewed by 16 bytes in shared memory), then the two runs of their scales.
 * Phase-2 tile (slab, chunk): the chunk's k-major rows, restricted to the slab's output columns. */
__device__ __forceinline__ void im_producer(const ImParams &P, ImSmem *sm, uint8_t *ring, int kb0, int kb1) {
    /* The whole warp: lane 0 waits for the stage and posts the byte count, then every lane issues one
     * of the tile's copies (a single thread issuing eighteen 2.5 KB copies per tile cannot keep up with
     * the HBM stream). */
    const int lane = threadIdx.x & 31;
    const int ns = P.nstages;
    const int nt1 = kb1 - kb0;
    int ckb[kImMaxChunks], cn[kImMaxChunks], cseg[kImMaxChunks], nseg = 0;
    const int nch = im_build_chunks(kb0, kb1, ckb, cn, cseg, &nseg);
    const int nt2 = nch * P.nslabs;
    const int Gs = P.G1; /* scales per gate/up row */
    int t = 0;
    bool failed = false;
    for (int l = 0; l < P.L && !failed; ++l) {
        const ImLayer &LY = P.layers[l];
        for (int lt = 0; lt < nt1 + nt2; ++lt, ++t) {
            const int s = t % ns;
            bool ok = true;
            if (lane == 0 && t >= ns) ok = mbar_wait<100>(&sm->empty[s], (uint32_t)(t / ns - 1) & 1u, &sm->abort_flag);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) im_give_up(sm, P.status, ST_PRODUCER_EMPTY);
                failed = true;
                break;
            }
            uint8_t *dst = ring + (size_t)s * P.stage_bytes;
            if (lt < nt1) {
                const int r0 = (kb0 + lt) * 8; /* first pair of the tile; 8 * Gs * 2 bytes of scales per run, 16-byte aligned */
                const uint32_t nsc = (uint32_t)(8 * Gs * 2);
                if (lane == 0) mbar_expect_tx(&sm->full[s], 16u * (uint32_t)P.rb1 + 2u * nsc);
                __syncwarp();
                if (lane < 8)
                    bulk_g2s(dst + (size_t)lane * P.rs1, LY.gu_w + (size_t)(r0 + lane) * P.rb1, (uint32_t)P.rb1, &sm->full[s]);
                else if (lane < 16)
                    bulk_g2s(dst + (size_t)lane * P.rs1, LY.gu_w + (size_t)(P.I + r0 + lane - 8) * P.rb1, (uint32_t)P.rb1, &sm->full[s]);
                else if (lane == 16)
                    bulk_g2s(dst + P.sc_off, (const uint8_t *)LY.gu_s + (size_t)r0 * Gs * 2, nsc, &sm->full[s]);
                else if (lane == 17)
                    bulk_g2s(dst + P.sc_off + P.sc_half_bytes, (const uint8_t *)LY.gu_s + (size_t)(r0 + P.I) * Gs * 2, nsc, &sm->full[s]);
            } else {
                const int tt = lt - nt1, sl = tt / nch, ch = tt % nch;
                const int c0 = sl * P.slab, cols = min(P.slab, P.H - c0);
                if (lane == 0) mbar_expect_tx(&sm->full[s], (uint32_t)cn[ch] * (uint32_t)cols * 4u);
                __syncwarp();
                if (lane < cn[ch])
                    bulk_g2s(dst + (size_t)lane * P.rs2, LY.wt + (size_t)(ckb[ch] + lane) * P.H + c0, (uint32_t)cols * 4u, &sm->full[s]);
            }
        }
    }
    if (lane == 0)
        for (int u = max(0, t - ns); u < t; ++u) { /* never leave with a copy of ours still in flight */
            bool done = false;
            for (uint32_t i = 0; i < kSpinLimit && !done; ++i) done = mbar_try_wait(&sm->full[u % ns], (uint32_t)(u / ns) & 1u);
            if (!done) atomicCAS(P.status, 0u, (unsigned)ST_DRAIN | ((unsigned)blockIdx.x << 8));
        }
}

/* ---- consumers: the layer's input ------------------------------------------------------------------ */
/* Loader threads (one per 32-element column chunk, the first H/32 consumer threads) fetch the first
 * layer's input before anything else happens ... */
template <int MT>
__device__ __forceinline__ void im_prefetch_input(const ImParams &P, uint32_t (&pre)[MT][16]) {
    const int ti = threadIdx.x - 32;
    const bool on = ti >= 0 && ti < P.H / 32;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint16_t *src = P.x + (size_t)m * P.H + (size_t)(on ? ti : 0) * 32;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 t4 = make_uint4(0, 0, 0, 0);
            if (on && m < P.M) t4 = __ldg((const uint4 *)(src + q * 8));
            pre[m][4 * q] = t4.x; pre[m][4 * q + 1] = t4.y; pre[m][4 * q + 2] = t4.z; pre[m][4 * q + 3] = t4.w;
        }
    }
}

/* ... and store 32 raw BF16 values per token into shared memory, with the sums of squares for a fused
 * RMSNorm; the loader warps then arrive at x_ready. */
template <int MT>
__device__ __forceinline__ void im_store_input(const ImParams &P, ImSmem *sm, uint16_t *xs, const uint32_t (&v)[MT][16]) {
    const int ti = threadIdx.x - 32, lane = threadIdx.x & 31, wp = ti >> 5;
    const bool loader = ti < P.H / 32;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        float ss = 0.0f;
        if (loader) {
            uint32_t *dst = (uint32_t *)(xs + (size_t)m * P.H + (size_t)ti * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q) *(uint4 *)(dst + 4 * q) = make_uint4(v[m][4 * q], v[m][4 * q + 1], v[m][4 * q + 2], v[m][4 * q + 3]);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                ss = fmaf(bf16_lo(v[m][q]), bf16_lo(v[m][q]), ss);
                ss = fmaf(bf16_hi(v[m][q]), bf16_hi(v[m][q]), ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) sm->norm_red[m][wp] = ss;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->x_ready);
}

/* Later layers: the input is the residual stream the previous layer's row owners published as tagged
 * words.  Returns false when a wait ran out. */
template <int MT>
__device__ __forceinline__ bool im_stage_input(const ImParams &P, ImSmem *sm, uint16_t *xs, int l) {
    const int ti = threadIdx.x - 32, lane = threadIdx.x & 31, wp = ti >> 5;
    const int loader_warps = (P.H / 32 + 31) / 32;
    if (l == 0 || wp >= loader_warps) return true;
    if (!mbar_wait<64>(&sm->h_open, (uint32_t)(l - 1) & 1u, &sm->abort_flag)) {
        if (lane == 0) im_give_up(sm, P.status, ST_NEXT_X);
        return false;
    }
    const unsigned tag = km_tag(sm->epoch + (unsigned)l - 1u); /* the previous layer's */
    const bool loader = ti < P.H / 32;
    uint32_t v[MT][16];
    bool bad = false;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int q = 0; q < 16; ++q) v[m][q] = 0;
        if (!loader || m >= P.M) continue;
        const unsigned long long *src = P.hx + (size_t)m * P.H + (size_t)ti * 32;
        bool in = false;
        for (uint32_t k = 0; k < kTpPollLimit && !in; ++k) {
            in = true;
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                unsigned long long a, b;
                km_load2(src + 2 * q, a, b);
                in = in && (unsigned)(a >> 32) == tag && (unsigned)(b >> 32) == tag;
                v[m][q] = ((unsigned)a >> 16) | ((unsigned)b & 0xFFFF0000u); /* the values are BF16-representable */
            }
            if (!in) {
                if ((k & 255u) == 255u && sm->abort_flag) break;
                __nanosleep(64);
            }
        }
        if (!in) bad = true;
    }
    if (__any_sync(0xffffffffu, bad)) { if (lane == 0) im_give_up(sm, P.status, ST_NEXT_X); return false; }
    im_store_input<MT>(P, sm, xs, v);
    return true;
}

/* The byte planes of the (normalized) input, built by all consumer threads: thread i takes the 8-code
 * words i, i + 544, ... of every token; the sixteen threads of a half-warp hold one 128-group and agree
 * on its exponent.  Layout: xp[((chunk * MT + token) * 2 + plane) * 32 + slot], plane 0 = hi, 1 = lo;
 * slot 4w+i = code 2i of word w of the 32-code chunk, slot 16+4w+i = code 2i+1 (the k order of the MMA's
 * A fragments built from word w). */
template <int MT>
__device__ __forceinline__ void im_build_planes(const ImParams &P, ImSmem *sm, const uint16_t *xs, uint8_t *xp, const ImLayer &LY) {
    const int ti = threadIdx.x - 32, lane = threadIdx.x & 31;
    const int words = P.H / 8;
    const bool normalize = LY.norm_w != nullptr;
    const float gemma = P.norm_gemma ? 1.0f : 0.0f;
    const int loader_warps = (P.H / 32 + 31) / 32;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        if (m >= P.M) break;
        float inv_rms = 1.0f;
        if (normalize) {
            float total = 0.0f;
            for (int w = 0; w < loader_warps; ++w) total += sm->norm_red[m][w];
            inv_rms = rsqrtf(total / (float)P.H + P.norm_eps);
        }
        for (int w0 = 0; w0 < words; w0 += kConsumerThreads) { /* uniform trip count; whole half-warps are in or out */
            const int w = w0 + ti;
            const bool on = w < words;
            float v[8];
            uint32_t mx = 0;
            {
                uint4 raw = make_uint4(0, 0, 0, 0), nw = make_uint4(0, 0, 0, 0);
                if (on) raw = *(const uint4 *)(xs + (size_t)m * P.H + (size_t)w * 8);
                if (on && normalize) nw = __ldg((const uint4 *)(LY.norm_w + (size_t)w * 8));
                const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w}, n4[4] = {nw.x, nw.y, nw.z, nw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float lo = bf16_lo(r[i]), hi = bf16_hi(r[i]);
                    if (normalize) { /* the reference's expression and its BF16 rounding */
                        lo = round_bf16(lo * inv_rms * (bf16_lo(n4[i]) + gemma));
                        hi = round_bf16(hi * inv_rms * (bf16_hi(n4[i]) + gemma));
                    }
                    v[2 * i] = lo; v[2 * i + 1] = hi;
                    mx = max(mx, __float_as_uint(lo) & 0x7FFFFFFFu);
                    mx = max(mx, __float_as_uint(hi) & 0x7FFFFFFFu);
                }
            }
            const unsigned hmask = 0xFFFFu << (lane & 16);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(hmask, mx, o));
            float up, fac;
            im_scaling((int)(mx >> 23), up, fac);
            if (on) {
                const uint4 pl = im_planes(v, up);
                const int chunk = w >> 2, wq = w & 3;
                uint8_t *base = xp + ((size_t)(chunk * MT + m) * 2) * 32;
                *(uint32_t *)(base + 4 * wq) = pl.x;           /* hi, even codes */
                *(uint32_t *)(base + 16 + 4 * wq) = pl.y;      /* hi, odd codes */
                *(uint32_t *)(base + 32 + 4 * wq) = pl.z;      /* lo, even */
                *(uint32_t *)(base + 32 + 16 + 4 * wq) = pl.w; /* lo, odd */
                if ((w & 15) == 0) sm->xfac[m][w >> 4] = fac;
            }
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm->xp_ready);
}

/* ---- epilogue warp: phase-1 sums -> act, then the byte planes of this CTA's act values ----------- */
template <int MT>
__device__ __forceinline__ bool im_epilogue_layer(const ImParams &P, ImSmem *sm, int l, int kb0, int kb1, int part_tile0,
                                                  unsigned &base) {
    constexpr int NVROW = 2 * MT;
    const int lane = threadIdx.x & 31;
    const int ntiles = kb1 - kb0;
    if (l == 0) {
        /* Both arrival counters stood at `base` when the launch began; `epoch` numbers the layers this
         * device has run (the tags); seq0 is the communicator's call number.  Read here, off everybody's
         * critical path, and published to the consumers by this warp's arrivals at act_ready / p_open. */
        unsigned b = 0;
        if (lane == 0) {
            b = P.sync[2];
            sm->base = b;
            sm->epoch = P.sync[3];
            sm->seq0 = P.tp > 1 ? ld_acquire_gpu(P.tp_seq) : 0u;
            sm->nchunks = im_build_chunks(kb0, kb1, sm->chunk_kb, sm->chunk_n, sm->chunk_seg, &sm->nseg);
        }
        base = __shfl_sync(0xffffffffu, b, 0);
    }
    /* the down projection's scale rows of this CTA's (at most two) groups for THIS layer: the buffer is
     * free, every consumer warp having stored the previous layer's partial sums (arrive_p) */
    if (lane == 0 && kb1 > kb0) {
        bool free_ = l == 0;
        for (uint32_t i = 0; i < kSpinLimit && !free_; ++i) {
            free_ = *(volatile unsigned *)&sm->arrive_p >= (unsigned)l * kConsumerWarps;
            if (!free_) { if ((i & 63) == 63 && sm->abort_flag) break; __nanosleep(64); }
        }
        if (free_) {
            const int g0 = kb0 / kImGroupKb, nseg = (kb1 - 1) / kImGroupKb - g0 + 1;
            uint8_t *st_s = (uint8_t *)sm + im_smem_header(MT) + P.xs_bytes + P.xp_bytes;
            mbar_expect_tx(&sm->st_full, (uint32_t)nseg * (uint32_t)P.H * 2u);
            for (int s = 0; s < nseg; ++s)
                bulk_g2s(st_s + (size_t)s * P.H * 2, P.layers[l].st + (size_t)(g0 + s) * P.H, (uint32_t)P.H * 2u, &sm->st_full);
        }
    }
    for (int lt = 0; lt < ntiles; ++lt) {
        const int pt = part_tile0 + lt;
        const int pslot = pt % kPartSlots;
        if (!mbar_wait<100>(&sm->part_full[pslot], (uint32_t)(pt / kPartSlots) & 1u, &sm->abort_flag)) {
            im_give_up(sm, P.status, ST_PART_FULL);
            return false;
        }
        const float *part = sm->part + (size_t)pslot * im_part_floats(MT);
        if (lane < 8 * MT) {
            const int p = lane / MT, m = lane % MT;
            const int row = (kb0 + lt) * 8 + p;
            float a = 0.0f, b = 0.0f;
            const float *pa = part + ((size_t)p * NVROW + m) * kImMaxParts;
            const float *pb = part + ((size_t)p * NVROW + MT + m) * kImMaxParts;
            for (int k = 0; k < P.nparts; ++k) { a += pa[k]; b += pb[k]; } /* warp order: fixed */
            const uint16_t v = f32_to_bf16_bits(silu_mul(round_bf16(a), round_bf16(b)));
            if (m < P.M) P.act[(size_t)m * P.I + row] = v;
            sm->act_s[m][lt * 8 + p] = v;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->part_empty[pslot]);
    }
    __syncwarp();
    /* one exponent per (token, group segment of this CTA's K range) */
    const int nseg = kb1 > kb0 ? (kb1 - 1) / kImGroupKb - kb0 / kImGroupKb + 1 : 0;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        for (int seg = 0; seg < nseg; ++seg) {
            const int g = kb0 / kImGroupKb + seg;
            const int lo = max(kb0, g * kImGroupKb), hi = min(kb1, (g + 1) * kImGroupKb);
            uint32_t mx = 0;
            for (int e = (lo - kb0) * 8 + lane; e < (hi - kb0) * 8; e += 32) mx = max(mx, (uint32_t)(sm->act_s[m][e] & 0x7FFFu));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float up, fac;
            im_scaling((int)(mx >> 7), up, fac);
            if (lane == 0) sm->afac[m][seg] = fac;
            const int kb = lo + lane;
            if (kb < hi) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = bf16_bits_to_f32(sm->act_s[m][(kb - kb0) * 8 + i]);
                *(uint4 *)sm->planes[m][kb - kb0] = im_planes(v, up);
            }
        }
    }
    __syncwarp();
    if (lane == 0 && kb1 > kb0) {
        mbar_arrive(&sm->act_ready);
        if (l == 0) im_stamp(P, 5);
    }
    /* idle until the next layer: watch the two arrival counters for the whole CTA (one poller per SM) */
    bool ok = true;
    if (lane == 0) {
        const unsigned target = base + (unsigned)(l + 1) * gridDim.x;
        ok = km_wait_counter(P.sync + 0, target, &sm->abort_flag);
        if (ok) {
            mbar_arrive(&sm->p_open);
            if (l == 0) im_stamp(P, 13);
            if (l + 1 < P.L) {
                ok = km_wait_counter(P.sync + 1, target, &sm->abort_flag);
                if (ok) mbar_arrive(&sm->h_open);
            }
        }
        if (!ok) im_give_up(sm, P.status, ST_PARTIALS);
    }
    return __shfl_sync(0xffffffffu, ok, 0);
}

/* ---- consumers: one layer ------------------------------------------------------------------------- */
template <int MT>
__device__ __forceinline__ bool im_consumer_layer(const ImParams &P, ImSmem *sm, uint16_t *xs, uint8_t *xp, const uint8_t *st_s,
                                                  uint8_t *ring, int l, int kb0, int kb1, int ring_tile0, int part_tile0) {
    constexpr int NVROW = 2 * MT;
    constexpr uint32_t kNib = 0xF0F0F0F0u;
    const ImLayer &LY = P.layers[l];
    const int stage_bytes = P.stage_bytes, nstages = P.nstages;
    const uint32_t ring_addr = smem_u32(ring), xp_addr = smem_u32(xp);
    const int ti = threadIdx.x - 32, lane = threadIdx.x & 31, wp = ti >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int G = (int)gridDim.x;
    const int nt1 = kb1 - kb0, nkb = kb1 - kb0;
    const int H = P.H;

    /* ---------------- the layer's input: raw values staged by the loaders, byte planes by everyone -- */
    if (!im_stage_input<MT>(P, sm, xs, l)) return false;
    if (!mbar_wait<32>(&sm->x_ready, (uint32_t)l & 1u, &sm->abort_flag)) {
        im_give_up(sm, P.status, ST_NEXT_X);
        return false;
    }
    im_build_planes<MT>(P, sm, xs, xp, LY);
    if (!mbar_wait<32>(&sm->xp_ready, (uint32_t)l & 1u, &sm->abort_flag)) {
        im_give_up(sm, P.status, ST_NEXT_X);
        return false;
    }
    if (threadIdx.x == 32 && l == 0) im_stamp(P, 2);

    /* ---------------- phase 1: one k-block of act per tile, K split over the warps ------------------ */
    const int grp0 = wp * P.gpp, grp1 = min(P.G1, grp0 + P.gpp);
    /* this lane's B fragment: column g = plane (g & 1) of token g / 2; columns beyond the tokens are zero */
    const bool bcol = g < 2 * MT;
    const uint32_t xp_lane = xp_addr + (uint32_t)(((g >> 1) * 2 + (g & 1)) * 32 + 4 * t);
    for (int lt = 0; lt < nt1; ++lt) {
        const int rt = ring_tile0 + lt, pt = part_tile0 + lt;
        const int s = rt % nstages;
        if (!mbar_wait<32>(&sm->full[s], (uint32_t)(rt / nstages) & 1u, &sm->abort_flag)) {
            im_give_up(sm, P.status, ST_CONSUMER_FULL);
            return false;
        }
        if (threadIdx.x == 32 && lt == 0 && l == 0) im_stamp(P, 3);
        const int pslot = pt % kPartSlots;
        if (pt >= kPartSlots) {
            if (!mbar_wait<100>(&sm->part_empty[pslot], (uint32_t)(pt / kPartSlots - 1) & 1u, &sm->abort_flag)) {
                im_give_up(sm, P.status, ST_PART_EMPTY);
                return false;
            }
        }
        if (wp < P.nparts) {
            const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)stage_bytes;
            const uint32_t wg = st + (uint32_t)g * (uint32_t)P.rs1 + 4u * (uint32_t)t;      /* gate row g, word t of a chunk */
            const uint32_t wu = wg + 8u * (uint32_t)P.rs1;                                   /* up row g */
            const uint32_t sg = st + (uint32_t)P.sc_off + (uint32_t)g * (uint32_t)P.G1 * 2u; /* their scale rows */
            const uint32_t su = sg + (uint32_t)P.sc_half_bytes;
            float vg = 0.0f, vu = 0.0f;
            for (int grp = grp0; grp < grp1; ++grp) {
                int d[4] = {0, 0, 0, 0};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t chunk = (uint32_t)(grp * 4 + c);
                    const uint32_t w0 = im_lds32(wg + chunk * 16u), w1 = im_lds32(wu + chunk * 16u);
                    uint32_t b0 = 0, b1 = 0;
                    if (bcol) {
                        b0 = im_lds32(xp_lane + chunk * (uint32_t)(MT * 64));
                        b1 = im_lds32(xp_lane + chunk * (uint32_t)(MT * 64) + 16u);
                    }
                    im_mma(d, (w0 << 4) & kNib, (w1 << 4) & kNib, w0 & kNib, w1 & kNib, b0, b1);
                }
                if (t < MT) { /* columns 2t, 2t+1 = {hi, lo} sums of token t: 16 * sum code * X of this group */
                    const float f = sm->xfac[t][grp];
                    vg = fmaf((float)(d[0] * 256 + d[1]), lds_bf16_at(sg + (uint32_t)grp * 2u) * f, vg);
                    vu = fmaf((float)(d[2] * 256 + d[3]), lds_bf16_at(su + (uint32_t)grp * 2u) * f, vu);
                }
            }
            if (t < MT) {
                float *part = sm->part + (size_t)pslot * im_part_floats(MT);
                part[((size_t)g * NVROW + t) * kImMaxParts + wp] = vg;
                part[((size_t)g * NVROW + MT + t) * kImMaxParts + wp] = vu;
            }
        }
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(&sm->empty[s]);
            mbar_arrive(&sm->part_full[pslot]);
        }
    }
    if (threadIdx.x == 32 && l == 0) im_stamp(P, 4);

    /* ---------------- phase 2: every output row against this CTA's own act values ------------------- */
    if (nkb > 0) {
        if (!mbar_wait<64>(&sm->act_ready, (uint32_t)l & 1u, &sm->abort_flag)) {
            im_give_up(sm, P.status, ST_ACT_READY);
            return false;
        }
        if (!mbar_wait<64>(&sm->st_full, (uint32_t)l & 1u, &sm->abort_flag)) {
            im_give_up(sm, P.status, ST_ACT_READY);
            return false;
        }
        if (threadIdx.x == 32 && l == 0) im_stamp(P, 6);
        /* (the launch's layer count and call number were read by the epilogue warp and are published by
         * its arrival at act_ready) */
        const unsigned tag = km_tag(sm->epoch + (unsigned)l);
        const int nch = sm->nchunks;
        const uint32_t st_addr = smem_u32(st_s);
        unsigned long long *mine = P.partial + (size_t)blockIdx.x * km_partial_stride(P.M, H);
        int tile = 0;
        for (int sl = 0; sl < P.nslabs; ++sl) {
            const int c0 = sl * P.slab, cols = min(P.slab, H - c0);
            const int nrb = cols / 16; /* 16-row blocks of this slab; warp w takes w, w + 17, ... */
            int d[kImMaxRb][4];
            float y[kImMaxRb][2];
#pragma unroll
            for (int i = 0; i < kImMaxRb; ++i) { d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0; y[i][0] = y[i][1] = 0.0f; }
            for (int ch = 0; ch < nch; ++ch, ++tile) {
                const int rt = ring_tile0 + nt1 + tile;
                const int s = rt % nstages;
                if (!mbar_wait<32>(&sm->full[s], (uint32_t)(rt / nstages) & 1u, &sm->abort_flag)) {
                    im_give_up(sm, P.status, ST_CONSUMER_FULL);
                    return false;
                }
                if (threadIdx.x == 32 && tile == 0 && l == 0) im_stamp(P, 7);
                const int n = sm->chunk_n[ch], seg = sm->chunk_seg[ch], kbf = sm->chunk_kb[ch] - kb0;
                /* B: lane (g, t) supplies k-block t of the chunk (zero beyond its n k-blocks), plane g & 1 of token g / 2 */
                uint32_t b0 = 0, b1 = 0;
                if (g < 2 * MT && t < n) {
                    const uint32_t *pl = sm->planes[g >> 1][kbf + t];
                    b0 = pl[(g & 1) * 2];       /* even codes */
                    b1 = pl[(g & 1) * 2 + 1];   /* odd codes */
                }
                const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)stage_bytes;
                const uint32_t wrow = st + (uint32_t)min(t, n - 1) * (uint32_t)P.rs2 + 4u * (uint32_t)g;
#pragma unroll
                for (int i = 0; i < kImMaxRb; ++i) {
                    const int rb = wp + kConsumerWarps * i;
                    if (rb < nrb) { /* uniform over the warp */
                        const uint32_t w0 = im_lds32(wrow + (uint32_t)rb * 64u), w1 = im_lds32(wrow + (uint32_t)rb * 64u + 32u);
                        im_mma(d[i], (w0 << 4) & kNib, (w1 << 4) & kNib, w0 & kNib, w1 & kNib, b0, b1);
                    }
                }
                if (ch == nch - 1 || sm->chunk_seg[ch + 1] != seg) { /* the group segment ends: scale its integer sums */
                    const float f = t < MT ? sm->afac[t][seg] : 0.0f;
                    const uint32_t sc = st_addr + (uint32_t)seg * (uint32_t)H * 2u + (uint32_t)(c0 + g) * 2u;
#pragma unroll
                    for (int i = 0; i < kImMaxRb; ++i) {
                        const int rb = wp + kConsumerWarps * i;
                        if (rb < nrb) {
                            if (t < MT) {
                                y[i][0] = fmaf((float)(d[i][0] * 256 + d[i][1]), lds_bf16_at(sc + (uint32_t)rb * 32u) * f, y[i][0]);
                                y[i][1] = fmaf((float)(d[i][2] * 256 + d[i][3]), lds_bf16_at(sc + (uint32_t)rb * 32u + 16u) * f, y[i][1]);
                            }
                            d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm->empty[s]);
            }
            /* this CTA's share of the slab's output rows, as tagged words: lane (g, t) holds rows g and g+8 of token t */
            if (t < P.M) {
#pragma unroll
                for (int i = 0; i < kImMaxRb; ++i) {
                    const int rb = wp + kConsumerWarps * i;
                    if (rb < nrb) {
                        unsigned long long *p = mine + (size_t)t * H + c0 + rb * 16 + g;
                        km_store1(p, km_word(y[i][0], tag));
                        km_store1(p + 8, km_word(y[i][1], tag));
                    }
                }
            }
        }
    }
    __syncwarp();
    if (lane == 0 && atomicAdd(&sm->arrive_p, 1u) % kConsumerWarps == kConsumerWarps - 1) km_arrive_counter(P.sync + 0); /* the CTA's last warp */
    if (threadIdx.x == 32 && l == 0) im_stamp(P, 8);

    /* ---------------- the rows this CTA owns: sum over CTAs, cross-rank exchange, output ------------ */
    /* Groups of eight lanes take one (row, token) item at a time.  Lane s adds the partial sums of the
     * CTAs s, s+8, ... in ascending order, a fixed three-step butterfly adds the eight lane sums (the
     * same bits in every lane), so the result does not depend on timing.  Under tensor parallelism
     * lane s then sends the rank's sum to ranks s (and s+8), waits for rank s's (and s+8's) word in
     * this rank's own buffer, and the values are added in rank order. */
    if (!mbar_wait<64>(&sm->p_open, (uint32_t)l & 1u, &sm->abort_flag)) {
        if (lane == 0) im_give_up(sm, P.status, ST_PARTIALS);
        return false;
    }
    if (threadIdx.x == 32 && l == 0) im_stamp(P, 10);
    const unsigned tag = km_tag(sm->epoch + (unsigned)l);
    const unsigned seq = sm->seq0 + (unsigned)l;
    const int MM = P.M;
    const int b2 = km_begin(H, blockIdx.x, G), e2 = km_begin(H, blockIdx.x + 1, G);
    const int nitems = (e2 - b2) * MM;
    const int s8 = lane & 7, grp8 = ti >> 3;
    constexpr int kGroups = kConsumerThreads / 8;
    const unsigned gmask = 0xFFu << (lane & 24);
    const int KB = P.I / 8;
    unsigned use_mask = 0; /* bit i: CTA s8 + 8i exists and owns k-blocks (a CTA without any stores nothing) */
    if (KB >= G) {
        for (int i = 0; i < kImMaxQ; ++i)
            if (s8 + 8 * i < G) use_mask |= 1u << i;
    } else {
        for (int i = 0; i < kImMaxQ; ++i) {
            const int q = s8 + 8 * i;
            if (q < G && km_begin(KB, q + 1, G) > km_begin(KB, q, G)) use_mask |= 1u << i;
        }
    }
    bool failed = false;
    for (int it0 = 0; it0 < nitems; it0 += kGroups) { /* uniform trip count over the CTA */
        const int item = it0 + grp8;
        const bool valid = item < nitems;
        const int ic = valid ? item : 0;
        const int row = b2 + ic / MM, m = ic % MM;
        unsigned long long w[kImMaxQ];
        bool in = false;
        for (uint32_t k = 0; k < kTpPollLimit && !in; ++k) {
            in = true;
#pragma unroll
            for (int i = 0; i < kImMaxQ; ++i) { /* all loads first, then the tag checks, so the loads overlap */
                w[i] = (unsigned long long)tag << 32;
                if ((use_mask >> i) & 1u) w[i] = km_load1(P.partial + (size_t)(s8 + 8 * i) * km_partial_stride(MM, H) + (size_t)m * H + row);
            }
#pragma unroll
            for (int i = 0; i < kImMaxQ; ++i) in = in && (unsigned)(w[i] >> 32) == tag;
            if (!in) {
                if ((k & 255u) == 255u && sm->abort_flag) break;
                __nanosleep(32);
            }
        }
        if (threadIdx.x == 32 && l == 0 && it0 == 0) im_stamp(P, 11);
        float a = 0.0f;
#pragma unroll
        for (int i = 0; i < kImMaxQ; ++i) a += __uint_as_float((unsigned)w[i]);
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
            const unsigned long long *own = P.peer_slots[P.rank] + (size_t)(seq & 1u) * P.tp * P.slot_stride + elem;
            float v[2] = {0.0f, 0.0f};
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r = s8 + 8 * u;
                if (r < P.tp && valid && !bad) {
                    const unsigned long long *p = own + (size_t)r * P.slot_stride;
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
            if (valid && s8 == 0) im_give_up(sm, P.status, partials_missing ? ST_PARTIALS : ST_PEER_DATA);
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
    if (threadIdx.x == 32 && l == 0) im_stamp(P, 9);
    return !failed;
}

/* ---- the kernel ----------------------------------------------------------------------------------- */
template <int MT>
__global__ void __launch_bounds__(kThreads, 1) ffn_imma_kernel(const __grid_constant__ ImParams P) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    ImSmem *sm = (ImSmem *)smem_raw;
    uint16_t *xs = (uint16_t *)(smem_raw + im_smem_header(MT));
    uint8_t *xp = (uint8_t *)xs + P.xs_bytes;
    uint8_t *st_s = xp + P.xp_bytes;
    uint8_t *ring = st_s + (size_t)kImMaxSeg * P.H * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0) {
        if (lane == 0) im_stamp(P, 0);
        if (lane < P.nstages) { mbar_init(&sm->full[lane], 1); mbar_init(&sm->empty[lane], kConsumerWarps); }
        if (lane >= 8 && lane < 8 + kPartSlots) { mbar_init(&sm->part_full[lane - 8], kConsumerWarps); mbar_init(&sm->part_empty[lane - 8], 1); }
        if (lane == 16) mbar_init(&sm->x_ready, (P.H / 32 + 31) / 32);
        if (lane == 17) mbar_init(&sm->act_ready, 1);
        if (lane == 18) mbar_init(&sm->p_open, 1);
        if (lane == 19) mbar_init(&sm->h_open, 1);
        if (lane == 20) { sm->arrive_p = 0; sm->arrive_h = 0; }
        if (lane == 21) mbar_init(&sm->xp_ready, kConsumerWarps);
        if (lane == 22) mbar_init(&sm->st_full, 1);
        if (lane == 31) sm->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        __syncwarp();
        /* the barriers exist: this warp (the producer) goes on at once, the others wait for it here */
        asm volatile("bar.arrive 1, %0;" ::"n"(kThreads) : "memory");
    } else {
        uint32_t pre[MT][16];
        im_prefetch_input<MT>(P, pre); /* in flight while warp 0 sets the barriers up */
        asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
        if (warp <= kConsumerWarps && (warp - 1) < (P.H / 32 + 31) / 32) im_store_input<MT>(P, sm, xs, pre);
    }
    const int G = (int)gridDim.x, KB = P.I / 8;
    const int kb0 = km_begin(KB, blockIdx.x, G), kb1 = km_begin(KB, blockIdx.x + 1, G);
    const int nt1 = kb1 - kb0;

    if (warp == 0) {
        if (lane == 0) im_stamp(P, 1);
        im_producer(P, sm, ring, kb0, kb1);
    } else if (warp <= kConsumerWarps) {
        /* phase-2 tiles per layer: chunks x slabs (the chunk count follows from the K range alone) */
        int ckb[kImMaxChunks], cn[kImMaxChunks], cseg[kImMaxChunks], nseg = 0;
        const int nt2 = im_build_chunks(kb0, kb1, ckb, cn, cseg, &nseg) * P.nslabs;
        for (int l = 0; l < P.L; ++l)
            if (!im_consumer_layer<MT>(P, sm, xs, xp, st_s, ring, l, kb0, kb1, l * (nt1 + nt2), l * nt1)) break;
    } else {
        unsigned base = 0;
        for (int l = 0; l < P.L; ++l)
            if (!im_epilogue_layer<MT>(P, sm, l, kb0, kb1, l * nt1, base)) break;
    }
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0 && !sm->abort_flag) {
        P.sync[2] = sm->base + (unsigned)P.L * (unsigned)G;
        P.sync[3] = sm->epoch + (unsigned)P.L;
        if (P.tp > 1) atomicAdd(P.tp_seq, (unsigned)P.L);
        im_stamp(P, 12);
    }
}

/* ============================================================================================= */
/* Host side                                                                                     */
/* ============================================================================================= */
static std::mutex g_im_mutex;
static bool g_im_attr_set[64][3];

/* Launch geometry from the shape alone.  `mt` is the token count padded to 1, 2 or 4 (the MMA's
 * column pairs).  Returns false when the kernel does not take the shape. */
static bool im_plan(ImParams &P, int tokens, int mt, int H, int I, int grid, int smem_optin, size_t &smem) {
    if (tokens < 1 || tokens > kImMaxTokens || mt < tokens) return false;
    if (H <= 0 || I <= 0 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP) return false;
    if (H / FFN_INT4_GROUP > kImMaxGroups || I > (1 << 22)) return false;
    if (grid < 1 || grid > 8 * kImMaxQ) return false;
    const int KB = I / 8;
    if ((KB + grid - 1) / grid > kImMaxKb) return false;
    P.M = tokens; P.H = H; P.I = I;
    P.G1 = H / FFN_INT4_GROUP;
    P.rb1 = H / 2; P.rs1 = P.rb1 + 16;
    P.gpp = (P.G1 + kImMaxParts - 1) / kImMaxParts;
    P.nparts = (P.G1 + P.gpp - 1) / P.gpp;
    P.sc_off = round_up(16 * P.rs1, 128);
    P.sc_half_bytes = round_up(8 * P.G1 * 2 + 32, 16);
    const int p1_stage = P.sc_off + 2 * P.sc_half_bytes;
    /* output rows per phase-2 slab: four chunk rows (slab * 4 + 32 bytes each) in about a phase-1 tile's room,
     * at most what 17 warps x kImMaxRb row blocks cover, a multiple of 32 (bank-conflict-free skew) */
    int slab = min(min((p1_stage / 4 - 32) / 4, kConsumerWarps * kImMaxRb * 16), H) / 32 * 32;
    if (slab < 32) return false;
    P.nslabs = (H + slab - 1) / slab;
    P.slab = round_up((H + P.nslabs - 1) / P.nslabs, 32);
    P.rs2 = P.slab * 4 + 32;
    P.stage_bytes = round_up(max(p1_stage, 4 * P.rs2), 128);
    P.xs_bytes = round_up(mt * H * 2, 128);
    P.xp_bytes = round_up(mt * H * 2, 128);
    const size_t fixed = im_smem_header(mt) + (size_t)P.xs_bytes + (size_t)P.xp_bytes + (size_t)kImMaxSeg * H * 2;
    if (fixed + 2 * (size_t)P.stage_bytes > (size_t)smem_optin) return false;
    P.nstages = (int)min((size_t)kMaxStages, ((size_t)smem_optin - fixed) / (size_t)P.stage_bytes);
    smem = fixed + (size_t)P.nstages * P.stage_bytes;
    return true;
}

static int im_padded_tokens(int tokens) { return tokens <= 1 ? 1 : tokens <= 2 ? 2 : 4; }

bool imma_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes) {
    static ImParams P; /* large: not on the stack */
    std::lock_guard<std::mutex> lock(g_im_mutex);
    P = ImParams();
    size_t smem = 0;
    if (!im_plan(P, tokens, im_padded_tokens(tokens), H, I, sm_count, smem_optin, smem)) return false;
    const int KB = I / 8;
    snprintf(out, out_bytes,
             "kernel=imma grid=%d threads=%d smem=%zu stages=%d stage_bytes=%d token_columns=%d p1_pairs_per_tile=8 p1_k_parts=%d "
             "p1_groups_per_part=%d p2_slab_rows=%d p2_slabs=%d kblocks_per_cta=%d..%d",
             sm_count, kThreads, smem, P.nstages, P.stage_bytes, im_padded_tokens(tokens), P.nparts, P.gpp, P.slab, P.nslabs,
             KB / sm_count, (KB + sm_count - 1) / sm_count);
    return true;
}

template <int MT>
static int im_launch(int dev, const ImParams &P, int grid, size_t smem, int smem_optin, cudaStream_t stream) {
    bool &set = g_im_attr_set[dev][MT == 1 ? 0 : MT == 2 ? 1 : 2];
    if (!set) {
        FFN_CUDA_TRY(cudaFuncSetAttribute(ffn_imma_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin),
                     "tensor-core decode FFN: shared-memory opt-in");
        set = true;
    }
    void *args[] = {(void *)&P};
    FFN_CUDA_TRY(cudaLaunchCooperativeKernel((const void *)ffn_imma_kernel<MT>, dim3(grid), dim3(kThreads), args, smem, stream),
                 "tensor-core decode FFN launch");
    return FFN_OK;
}

static_assert(sizeof(ImParams) <= 4000, "the kernel parameters must fit the 4 KB parameter space");

/* Same contract as kmajor_ffn_launch (kernels.h), for 1..4 tokens. */
int imma_ffn_launch(cudaStream_t stream, const void *x, void *act, void *layer_out, const FfnMlpWeights *layers,
                    int num_layers, int tokens, int H, int I, const FusedTp *tp, void *residual, int with_norm,
                    float eps, int gemma, unsigned *status) {
    if (tokens < 1 || tokens > kImMaxTokens || num_layers < 1) return FFN_NOT_ADMITTED;
    if (num_layers > 1 && (residual != x || !with_norm)) return FFN_NOT_ADMITTED;
    int dev = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return FFN_NOT_ADMITTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)act & 1)) return FFN_NOT_ADMITTED;
    KmDeviceView d;
    const int st = kmajor_device_view(H, tokens, &d);
    if (st) return st;
    if (!d.cooperative) return FFN_NOT_ADMITTED;
    std::lock_guard<std::mutex> lock(g_im_mutex);
    static ImParams P; /* 3 KB; guarded by the mutex above */
    P = ImParams();
    size_t smem = 0;
    const int mt = im_padded_tokens(tokens);
    const int grid = d.sm_count; /* under TP every rank runs the same grid: CTA c owns the same rows everywhere */
    if (!im_plan(P, tokens, mt, H, I, grid, d.smem_optin, smem)) return FFN_NOT_ADMITTED;
    for (int l = 0; l < num_layers; ++l) { /* all or nothing, before anything is launched */
        const uint32_t *wt; const uint16_t *sc;
        if (!kmajor_lookup(layers[l].down_i4, H, I, dev, &wt, &sc)) return FFN_NOT_ADMITTED;
        if (((uintptr_t)layers[l].gate_up_i4 & 15) || ((uintptr_t)layers[l].gate_up_i4_scales & 15)) return FFN_NOT_ADMITTED;
        if (with_norm && (!layers[l].post_norm_w || ((uintptr_t)layers[l].post_norm_w & 15))) return FFN_NOT_ADMITTED;
    }
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
        if (tokens * H > tp->slot_stride) return fail(FFN_ERR_CONFIG, "tensor-core decode FFN: %d tokens exceed the exchange buffer", tokens);
    }
    P.norm_eps = eps; P.norm_gemma = gemma;
    P.trace = fused_get_trace();
    for (int l0 = 0; l0 < num_layers; l0 += kImMaxLayers) {
        P.L = min(kImMaxLayers, num_layers - l0);
        for (int l = 0; l < P.L; ++l) {
            const FfnMlpWeights &w = layers[l0 + l];
            const uint32_t *wt = nullptr; const uint16_t *sc = nullptr;
            (void)kmajor_lookup(w.down_i4, H, I, dev, &wt, &sc);
            P.layers[l] = {w.gate_up_i4, (const uint16_t *)w.gate_up_i4_scales, wt, sc, with_norm ? (const uint16_t *)w.post_norm_w : nullptr};
        }
        int rc;
        if (mt == 1) rc = im_launch<1>(dev, P, grid, smem, d.smem_optin, stream);
        else if (mt == 2) rc = im_launch<2>(dev, P, grid, smem, d.smem_optin, stream);
        else rc = im_launch<4>(dev, P, grid, smem, d.smem_optin, stream);
        if (rc) return rc;
    }
    return FFN_OK;
}

}  // namespace ffn
