/*
 * ffn_tc.cu - the batched INT4 FFN (3 <= M <= 64 tokens per pass) on the fifth-generation tensor
 * cores: tcgen05.mma with the accumulators in tensor memory.
 *
 * The reference keeps every M > 1 on cuBLAS BF16 over a dequantized copy of the weights
 * (csrc/kernels/layers.cu:120-126); here the packed INT4 rows stay the only weight traffic.
 *
 *   swap-AB: 128 WEIGHT rows fill the MMA's M dimension (one row per tensor-memory lane), the tokens,
 *   padded to a multiple of 16, its N dimension.  Per 128-wide quantization group the tensor core
 *   accumulates  sum code * x  in FP32 (codes are exact in BF16, products exact), and the epilogue
 *   multiplies that partial sum by the group's scale and adds it to an FP32 register - the arithmetic
 *   of the reference's tiled kernel (csrc/kernels/gemm_quant.cu:134-147), so dequantization is exact.
 *
 * Roles of a CTA (one per SM, persistent over its units of 128 rows):
 *   warps 0-3   epilogue: tcgen05.ld of a finished group (warp w reads lanes 32w..32w+31: thread =
 *               weight row), scale, accumulate; at the end of a unit SiLU(gate)*up or the split-K
 *               hand-over and the output / cross-rank exchange.
 *   warp 4      producer (one thread): per stage two tiled TMA loads (cp.async.bulk.tensor.2d, 64 rows x
 *               128 bytes of packed codes each, 128-byte swizzle so the conversion warps read without
 *               bank conflicts) and one bulk copy of the stage's slice of the activations, completion
 *               on mbarriers; the ring is as deep as shared memory allows (4 to 8 stages).
 *   warps 5-12  conversion: INT4 codes of the stage -> exact BF16 codes, written from registers straight
 *               into tensor memory (tcgen05.st), where the MMA reads its A operand: no shared-memory
 *               copy of the 4x larger BF16 tile, so shared memory is all ring.  Two teams of four
 *               warps (one warp per tensor-memory quadrant) take alternate stages.
 *   warps 13-16 one thread each issues the MMAs (8 per group, K = 16, A from tensor memory, B = the
 *               stage's activation slice in shared memory) of every fourth group and commits them to
 *               the mbarriers that publish the accumulator and free the operands; warp 13 also
 *               allocates and frees tensor memory.
 * Tensor memory (512 columns): four accumulators of N FP32 columns and four operand buffers of 64
 * columns; group g uses accumulator, operand buffer and barriers g mod 4, so the MMAs of the next
 * groups run while group g is read out and group g+4 is converted.
 *
 * Activations are read in "tile order": K in blocks of 64 values; within a block token n owns a
 * 128-byte row at (n/8)*1024 + (n%8)*128 whose 16-byte piece c (8 values of K) sits at piece c ^ (n%8),
 * the 8 values in the order (0,4),(1,5),(2,6),(3,7) - the order in which one lop3 + one packed subtract
 * deliver the codes of a 32-bit word.  A stage's slice is then one contiguous bulk copy and already
 * the MMA's swizzled B-operand layout.  A small pre-pass writes the input that way; the gate/up
 * epilogue writes act that way for the down launch (and in natural order for the caller).
 *
 * Two launches per FFN, as the mma.sync pair (ffn_mma.cu): gate/up + SiLU*up, then down with K split
 * over CTAs (FP32 partial sums through global memory, added in split order by the last to arrive) and
 * the cross-rank exchange in its epilogue (tagged words, as the decode kernel).
 * Every wait is bounded; a wait that runs out records where, and every thread still reaches the end of
 * the kernel, where tensor memory is released.
 */
#include <stdio.h>

#include <mutex>

#include <cuda.h>
#include <cudaTypedefs.h>

#include "kernels.h"
#include "stream_common.cuh"

namespace ffn {

constexpr int kTcRows = 128;                  /* weight rows per unit = the MMA's M = tensor-memory lanes */
constexpr int kTcGroupsPerStage = 2;
constexpr int kTcGroupBytes = FFN_INT4_GROUP / 2;                       /* 64 packed bytes per row and group */
constexpr int kTcRowPitch = kTcGroupsPerStage * kTcGroupBytes;          /* 128: one row of a stage = the TMA box's inner extent = the 128-byte swizzle span */
constexpr int kTcMaxStages = 8;               /* ring of packed stages: as many as shared memory holds, at most 8 */
constexpr int kTcABufs = 4;                   /* converted operand buffers in tensor memory, one per MMA-issuing thread */
constexpr int kTcAccBufs = 4;
constexpr int kTcACols = FFN_INT4_GROUP / 2;  /* 64 columns of tensor memory hold one group of a row in BF16 (two values per column) */
constexpr int kTcAFirstCol = 256;             /* columns 0..255: 4 accumulators of up to 64 FP32 columns; 256..511: 4 operand buffers */
constexpr int kTcTmemCols = 512;
constexpr int kTcEpiWarps = 4, kTcConvWarps = 8, kTcMmaWarps = 4;
constexpr int kTcConvTeams = 2;               /* conversion teams of 4 warps: team t converts the stages with index = t mod 2 */
constexpr int kTcTeamWarps = kTcConvWarps / kTcConvTeams;
constexpr int kTcProducerWarp = kTcEpiWarps, kTcFirstConvWarp = kTcEpiWarps + 1, kTcFirstMmaWarp = kTcFirstConvWarp + kTcConvWarps;
constexpr int kTcThreads = (kTcFirstMmaWarp + kTcMmaWarps) * 32;        /* 544 */
constexpr int kTcMaxSplits = 8;
constexpr int kTcHeader = 9216;               /* barriers, flags, the two 64 x 17 hand-over buffers of the pairs epilogue */
constexpr int kTcScaleGroups = 64;            /* groups of scales the epilogue keeps in shared memory at a time: [64][128 rows] bf16 */
constexpr int kTcScaleBytes = kTcScaleGroups * kTcRows * 2;
constexpr int kTcBoxRows = 64;                /* rows per TMA box: the gate half and the up half of a unit are separate row ranges */

/* where a bounded wait gave up (status word, low byte), continuing the decode kernels' numbering */
enum { ST_TC_STAGE_EMPTY = 20, ST_TC_STAGE_FULL = 21, ST_TC_A_EMPTY = 22, ST_TC_A_READY = 23, ST_TC_D_EMPTY = 24, ST_TC_D_FULL = 25 };
static_assert(kTcABufs == kTcAccBufs, "group g uses operand buffer, accumulator and `done` barrier g mod 4");

struct TcSmem {
    uint64_t full[kTcMaxStages], empty[kTcMaxStages];
    uint64_t a_ready[kTcABufs];             /* a converted operand buffer is complete (one arrival per warp of the team) */
    uint64_t done[kTcAccBufs];              /* the MMAs of a group have completed: its accumulator can be read, its operand buffer reused */
    uint64_t d_empty[kTcAccBufs];           /* the epilogue has read the accumulator out */
    uint32_t tmem_base;
    int abort_flag;
    int last_arrival;
    float ex_gate[64 * 17], ex_up[64 * 17]; /* the pairs epilogue's hand-over, 16 tokens at a time */
};
static_assert(sizeof(TcSmem) <= kTcHeader, "header");

struct TcParams {
    CUtensorMap wmap;         /* the packed rows [rows][K/2] as a 2-D byte tensor, box 128 bytes x 64 rows, 128-byte swizzle */
    const uint8_t *xt;        /* activations in tile order */
    const uint16_t *s;        /* scales [rows][K/128] */
    int M, npad;              /* tokens; tokens padded to a multiple of 16 */
    int N, K;                 /* pairs launch: gate/up pairs of this rank; down launch: output rows.  K: columns */
    int up_offset;            /* pairs launch: row of up row 0 */
    int units, splits;        /* units of 128 rows (x K splits for the down launch) */
    int stages;               /* depth of the packed ring */
    uint16_t *act;            /* pairs: bf16 [M][N] natural order */
    uint8_t *act_t;           /* pairs: the same in tile order (input of the down launch) */
    uint16_t *out;            /* down: bf16 [M][N] */
    uint16_t *residual;       /* down: optional bf16 [M][N], h <- bf16(h + y) */
    float *partial;           /* down: [splits][M][N] fp32 */
    unsigned *arrivals;       /* down: [N / 128], zero between launches */
    int tp, rank, slot_stride;
    unsigned long long *const *peer_slots;
    unsigned *tp_seq;
    unsigned *status;         /* word 3 of the device's synchronisation words */
    long long *trace;         /* debugging aid (ffn_int4_debug_trace): CTA 0 stamps the first 64 groups of each role */
};

/* role r, group gi -> trace[r * 64 + gi], SM clock cycles; role 7 holds single events (0: epilogue starts a
 * unit, 1: its group loop is over, 2: the unit's output is written) */
__device__ __forceinline__ void tc_stamp(const TcParams &P, int role, uint32_t gi) {
    if (P.trace && blockIdx.x == 0 && gi < 64u) P.trace[role * 64 + gi] = clock64();
}

/* ---- tcgen05 wrappers ------------------------------------------------------------------------ */
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
/* D[tmem] (+)= A[tmem] * B[smem]: M = 128 (lane = row), N and the operand types from the instruction
 * descriptor, K = 16; one column of A = two consecutive values of K in BF16 */
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
/* 16 consecutive columns of this thread's lane */
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
/* 16 consecutive FP32 columns of this thread's lane */
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&d)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]),
                   "=r"(d[8]), "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
                 : "r"(taddr));
}
/* tiled TMA load of one box: x = byte offset within the row (a multiple of 16), y = row */
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); } /* the four epilogue warps */

/* Shared-memory operand descriptor: K-major, 128-byte swizzle.  A row of the operand is 128 bytes (64
 * values of K); 8 rows form a 1024-byte atom inside which the 16-byte piece c of row r sits at piece
 * c ^ (r & 7); `sbo` is the distance between 8-row atoms.  The leading-dimension field is not used by
 * swizzled K-major layouts (set to 1, as CUTLASS does); bits 46-47 = 1 is the descriptor version of this
 * architecture, layout type 2 (bits 61-63) the 128-byte swizzle.  An MMA's K = 16 (32 bytes) is
 * selected inside the 128-byte row by adding 32 bytes to the start address. */
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t sbo) {
    const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}
/* Instruction descriptor of kind::f16: D = FP32 (bits 4-5 = 1), A = B = BF16 (bits 7-9, 10-12 = 1), both
 * K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28. */
__device__ __forceinline__ uint32_t tc_instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
}
/* nibbles s and s+4 of a word as exact BF16 codes (low half: nibble s, high half: nibble s+4):
 * 0x4300 | n is 128 + n, the xor with 8 turns the two's-complement nibble into code + 8 */
__device__ __forceinline__ uint32_t tc_codes(uint32_t w_shifted) {
    uint32_t v, d;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43084308, 0x6A;" : "=r"(v) : "r"(w_shifted));
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(v), "r"(0x43084308u));
    return d;
}
__device__ __forceinline__ int tc_permute8(int e) { return ((e & 3) << 1) | (e >> 2); }
/* byte offset of token n's 16-byte piece c inside one K block of the activations' tile order */
__host__ __device__ __forceinline__ int tc_tile_offset(int n, int c) { return (n >> 3) * 1024 + (n & 7) * 128 + ((c ^ (n & 7)) << 4); }

/* Bounded wait of a whole warp: one lane polls, the result reaches the others through a shuffle (which
 * also orders their later accesses after the poll).  Thirty-two lanes polling the same barrier word
 * only multiply the shared-memory traffic that every other warp's loads and arrivals queue behind. */
__device__ __forceinline__ bool tc_warp_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait<32>(bar, parity, abort_flag) ? 1 : 0;
    return __shfl_sync(~0u, ok, 0) != 0;
}

struct TcUnit {
    int row_a, row_b;   /* weight rows of lanes 0-63 and 64-127 */
    int g0, g1;         /* quantization groups of K this unit covers */
    int rb, sp;         /* down: row block and K split */
};
template <bool PAIRS>
__device__ __forceinline__ TcUnit tc_unit(const TcParams &P, int u) {
    TcUnit t;
    const int G = P.K / FFN_INT4_GROUP;
    if (PAIRS) {
        t.row_a = u * 64; t.row_b = P.up_offset + u * 64; t.g0 = 0; t.g1 = G; t.rb = u; t.sp = 0;
    } else {
        t.rb = u / P.splits; t.sp = u % P.splits;
        t.row_a = t.rb * kTcRows; t.row_b = t.row_a + 64;
        /* split boundaries on multiples of 8 groups where the split is long enough: the epilogue then
         * fetches its row's scales with 16-byte loads */
        t.g0 = (int)((long long)G * t.sp / P.splits); t.g1 = (int)((long long)G * (t.sp + 1) / P.splits);
        if (G >= 16 * P.splits) {
            if (t.sp > 0) t.g0 = (t.g0 + 4) & ~7;
            if (t.sp + 1 < P.splits) t.g1 = (t.g1 + 4) & ~7;
        }
    }
    return t;
}
__device__ __forceinline__ void tc_give_up(TcSmem *sm, unsigned *status, int where) {
    sm->abort_flag = 1;
    atomicCAS(status, 0u, (unsigned)where | ((unsigned)blockIdx.x << 8));
}

/* The down launch's output for one weight row: through the exchange slots when tensor parallel, else
 * straight to the caller's buffers (as the mma.sync pair's epilogue). */
template <int NPAD>
__device__ __forceinline__ void tc_down_output(const TcParams &P, TcSmem *sm, const float (&acc)[NPAD], int grow, unsigned seq) {
    if (P.tp > 1) {
        const size_t slot = (size_t)((seq & 1u) * P.tp + P.rank) * P.slot_stride;
#pragma unroll
        for (int m = 0; m < NPAD; ++m)
            if (m < P.M)
                for (int q = 0; q < P.tp; ++q) tp_store_tagged(P.peer_slots[q] + slot + (size_t)m * P.N + grow, acc[m], tp_tag(seq));
        const unsigned long long *mine = P.peer_slots[P.rank] + (size_t)(seq & 1u) * P.tp * P.slot_stride;
        for (int m = 0; m < P.M; ++m) {
            const size_t o = (size_t)m * P.N + grow;
            float y = 0.0f;
            if (!tp_wait_sum(mine + o, (size_t)P.slot_stride, P.tp, tp_tag(seq), &sm->abort_flag, 40, &y)) {
                tc_give_up(sm, P.status, ST_PEER_DATA);
                break;
            }
            const float v = round_bf16(y);
            P.out[o] = f32_to_bf16_bits(v);
            if (P.residual) P.residual[o] = f32_to_bf16_bits(bf16_bits_to_f32(P.residual[o]) + v);
        }
    } else {
#pragma unroll
        for (int m = 0; m < NPAD; ++m)
            if (m < P.M) {
                const size_t o = (size_t)m * P.N + grow;
                const float v = round_bf16(acc[m]);
                P.out[o] = f32_to_bf16_bits(v);
                if (P.residual) P.residual[o] = f32_to_bf16_bits(bf16_bits_to_f32(P.residual[o]) + v);
            }
    }
}

template <int NT, bool PAIRS>
__global__ void __launch_bounds__(kTcThreads, 1) ffn_tc_kernel(const __grid_constant__ TcParams P) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    TcSmem *sm = (TcSmem *)smem_raw;
    uint16_t *sc_t = (uint16_t *)(smem_raw + kTcHeader); /* the epilogue's scales: [group][row] */
    uint8_t *ring = smem_raw + kTcHeader + kTcScaleBytes;
    const uint32_t nstages = (uint32_t)P.stages;
    constexpr int NPAD = NT * 16;
    constexpr int kStageBytes = kTcRows * kTcRowPitch + kTcGroupsPerStage * NPAD * 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == kTcProducerWarp && lane == 0) {
        for (int i = 0; i < kTcMaxStages; ++i) { mbar_init(&sm->full[i], 1); mbar_init(&sm->empty[i], kTcTeamWarps + kTcGroupsPerStage); }
        for (int i = 0; i < kTcABufs; ++i) mbar_init(&sm->a_ready[i], kTcTeamWarps);
        for (int i = 0; i < kTcAccBufs; ++i) { mbar_init(&sm->done[i], 1); mbar_init(&sm->d_empty[i], kTcEpiWarps); }
        sm->abort_flag = 0;
        sm->last_arrival = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcFirstMmaWarp) {
        tmem_alloc(&sm->tmem_base, kTcTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm->tmem_base;
    /* the call's number, read by the down launch (slot parity and tag of the exchanged words) */
    if (PAIRS && blockIdx.x == 0 && threadIdx.x == 0 && P.tp_seq) atomicAdd(P.tp_seq, 1u);

    if (warp == kTcProducerWarp) {
        /* ---------------- producer (one thread) ---------------- */
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < P.units && ok; u += gridDim.x) {
                const TcUnit t = tc_unit<PAIRS>(P, u);
                for (int g = t.g0; g < t.g1; g += kTcGroupsPerStage, ++it) {
                    const int ng = min(kTcGroupsPerStage, t.g1 - g);
                    const uint32_t slot = it % nstages;
                    if (it >= nstages && !mbar_wait<64>(&sm->empty[slot], (it / nstages - 1) & 1u, &sm->abort_flag)) {
                        tc_give_up(sm, P.status, ST_TC_STAGE_EMPTY);
                        ok = false;
                        break;
                    }
                    uint8_t *dst = ring + (size_t)slot * kStageBytes;
                    /* a box is always two groups wide: at an odd tail the second half is the row's next
                     * bytes or, past the row's end, the fill value - nobody reads it */
                    const uint32_t x_bytes = (uint32_t)ng * NPAD * 256;
                    mbar_expect_tx(&sm->full[slot], kTcRows * kTcRowPitch + x_bytes);
                    tma_load_2d(dst, &P.wmap, g * kTcGroupBytes, t.row_a, &sm->full[slot]);
                    tma_load_2d(dst + kTcBoxRows * kTcRowPitch, &P.wmap, g * kTcGroupBytes, t.row_b, &sm->full[slot]);
                    bulk_g2s(dst + kTcRows * kTcRowPitch, P.xt + (size_t)g * NPAD * 256, x_bytes, &sm->full[slot]);
                    tc_stamp(P, 0, it);
                }
            }
            /* never leave with a copy of ours in flight: wait (bounded) for the most recent fill of every stage */
            for (uint32_t f = it > nstages ? it - nstages : 0u; f < it; ++f) {
                bool done = false;
                for (uint32_t i = 0; i < kSpinLimit && !done; ++i) done = mbar_try_wait(&sm->full[f % nstages], (f / nstages) & 1u);
                if (!done) atomicCAS(P.status, 0u, (unsigned)ST_DRAIN | ((unsigned)blockIdx.x << 8));
            }
        }
        __syncwarp();
    } else if (warp >= kTcFirstConvWarp && warp < kTcFirstMmaWarp) {
        /* ---------------- conversion: INT4 -> BF16 operand tiles ---------------- */
        /* Two teams of four warps; team t converts the stages whose running index is t mod 2 (both groups
         * of the stage, so the barrier traffic is paid once per stage), and the two teams work on two
         * stages at a time.  A thread owns one weight row = one lane of tensor memory; a warp reaches
         * the 32 lanes of quadrant (warp index mod 4), and the four warps of a team cover the four
         * quadrants.  The converted row (64 columns = 128 BF16 codes per group) goes straight from
         * registers to tensor memory, where the MMA reads its A operand. */
        const int cw = warp - kTcFirstConvWarp;
        const uint32_t team = (uint32_t)(cw / kTcTeamWarps);
        const int row = (warp & 3) * 32 + lane;
        const uint32_t a_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)kTcAFirstCol;
        const bool stamps = lane == 0 && (cw % kTcTeamWarps) == 0;
        uint32_t it = 0, gi = 0, slot = 0, round = 0; /* slot = it mod stages, round = it div stages */
        bool ok = true;
        for (int u = blockIdx.x; u < P.units && ok; u += gridDim.x) {
            const TcUnit t = tc_unit<PAIRS>(P, u);
            for (int g = t.g0; g < t.g1 && ok; g += kTcGroupsPerStage) {
                const int ng = min(kTcGroupsPerStage, t.g1 - g);
                if ((it & 1u) == team) {
                    ok = tc_warp_wait(&sm->full[slot], round & 1u, &sm->abort_flag, lane); /* tcgen05.st is warp-wide: the warp goes on together or not at all */
                    if (!ok) {
                        if (lane == 0) tc_give_up(sm, P.status, ST_TC_STAGE_FULL);
                        break;
                    }
                    /* 128-byte swizzle: 16-byte piece c of row r sits at piece c ^ (r & 7) of the row */
                    const uint32_t src0 = smem_u32(ring + (size_t)slot * kStageBytes) + (uint32_t)(row * kTcRowPitch);
                    for (int k = 0; k < ng; ++k) {
                        const uint32_t gk = gi + (uint32_t)k, ab = gk % kTcABufs;
                        /* the buffer was last read by the MMAs of group gk - 4, whose `done` barrier is this group's too */
                        if (gk >= (uint32_t)kTcABufs) {
                            ok = tc_warp_wait(&sm->done[ab], (gk / kTcABufs - 1) & 1u, &sm->abort_flag, lane);
                            if (!ok) {
                                if (lane == 0) tc_give_up(sm, P.status, ST_TC_A_EMPTY);
                                break;
                            }
                            tc_fence_after();
                        }
                        if (stamps) tc_stamp(P, 1, gk);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 wv = lds16_at(src0 + (uint32_t)((((k << 2) + q) ^ (row & 7)) << 4));
                            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
                            uint32_t v[16];
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const uint32_t w = words[c];
                                v[4 * c + 0] = tc_codes(w); v[4 * c + 1] = tc_codes(w >> 4);
                                v[4 * c + 2] = tc_codes(w >> 8); v[4 * c + 3] = tc_codes(w >> 12);
                            }
                            tmem_st16(a_lane + ab * (uint32_t)kTcACols + (uint32_t)(q * 16), v);
                        }
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sm->a_ready[ab]);
                        if (stamps) tc_stamp(P, 2, gk);
                    }
                    if (!ok) break;
                    if (lane == 0) mbar_arrive(&sm->empty[slot]); /* this warp is done with the stage's packed rows */
                }
                gi += (uint32_t)ng;
                ++it;
                if (++slot == nstages) { slot = 0; ++round; }
            }
        }
    } else if (warp >= kTcFirstMmaWarp) {
        /* ---------------- MMA issue: one thread per accumulator buffer ---------------- */
        /* Thread w issues the MMAs of the groups whose running index is w mod 4 into accumulator w, so
         * the fixed cost of issuing (barrier polls, eight MMAs, two commits) is paid by four threads
         * in turn; the tensor core takes the groups in whatever order they arrive - they are independent. */
        const uint32_t mine = (uint32_t)(warp - kTcFirstMmaWarp);
        if (lane == 0) {
            const uint32_t idesc = tc_instr_desc(NPAD);
            const uint64_t bdesc0 = tc_smem_desc(smem_u32(ring) + kTcRows * kTcRowPitch, 1024);
            const uint32_t dcol = tmem + mine * (uint32_t)NPAD, acol = tmem + (uint32_t)kTcAFirstCol + mine * (uint32_t)kTcACols;
            uint32_t it = 0, gi = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < P.units && ok; u += gridDim.x) {
                const TcUnit t = tc_unit<PAIRS>(P, u);
                for (int g = t.g0; g < t.g1 && ok; g += kTcGroupsPerStage, ++it) {
                    const int ng = min(kTcGroupsPerStage, t.g1 - g);
                    const uint32_t slot = it % nstages;
                    for (int k = 0; k < ng; ++k, ++gi) {
                        if (gi % kTcAccBufs != mine) continue;
                        if (!mbar_wait<20>(&sm->full[slot], (it / nstages) & 1u, &sm->abort_flag)) {
                            tc_give_up(sm, P.status, ST_TC_STAGE_FULL);
                            ok = false;
                            break;
                        }
                        if (!mbar_wait<20>(&sm->a_ready[mine], (gi / kTcABufs) & 1u, &sm->abort_flag)) {
                            tc_give_up(sm, P.status, ST_TC_A_READY);
                            ok = false;
                            break;
                        }
                        if (gi >= (uint32_t)kTcAccBufs && !mbar_wait<20>(&sm->d_empty[mine], (gi / kTcAccBufs - 1) & 1u, &sm->abort_flag)) {
                            tc_give_up(sm, P.status, ST_TC_D_EMPTY);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        tc_stamp(P, 3, gi);
                        /* descriptors differ from the first stage's only in the start-address field (bytes / 16) */
                        const uint64_t bdesc = bdesc0 + (uint64_t)((slot * (uint32_t)kStageBytes + (uint32_t)(k * NPAD * 256)) >> 4);
#pragma unroll
                        for (int i = 0; i < FFN_INT4_GROUP / 16; ++i)
                            tc_mma_ts(dcol, acol + (uint32_t)(i * 8), /* K = 16 is 8 columns of A */
                                      bdesc + (uint64_t)(((i >> 2) * NPAD * 128 + (i & 3) * 32) >> 4), idesc, i > 0 ? 1u : 0u);
                        tc_commit(&sm->done[mine]);      /* the sums are in tensor memory and the operand buffer is free */
                        tc_commit(&sm->empty[slot]);     /* this group's half of the stage's activation slice has been read */
                        if (ng < kTcGroupsPerStage) tc_commit(&sm->empty[slot]); /* an odd tail: the arrival of the group that is not there */
                        tc_stamp(P, 4, gi);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        /* ---------------- epilogue (warps 0-3: thread = tensor-memory lane = weight row) ---------------- */
        const int L = threadIdx.x;
        const int G = P.K / FFN_INT4_GROUP;
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        const unsigned seq = (!PAIRS && P.tp > 1) ? (*(volatile unsigned *)P.tp_seq - 1u) : 0u;
        uint32_t gi = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < P.units; u += gridDim.x) {
            const TcUnit t = tc_unit<PAIRS>(P, u);
            const int grow = L < 64 ? t.row_a + L : t.row_b + (L - 64);
            const uint16_t *srow = P.s + (size_t)grow * G;
            float acc[NPAD];
#pragma unroll
            for (int c = 0; c < NPAD; ++c) acc[c] = 0.0f;
            ok = __all_sync(~0u, ok && !sm->abort_flag);
            if (L == 0 && u == (int)blockIdx.x) tc_stamp(P, 7, 0);
            /* The scales of this row come through shared memory, 64 groups at a time: a global load per
             * group would put its latency (hundreds of cycles) into every turn of the loop below.  A
             * thread reads back only what it wrote itself, so no barrier is needed. */
            for (int gc = t.g0; gc < t.g1; gc += kTcScaleGroups) {
                const int nc = min(kTcScaleGroups, t.g1 - gc);
                int j = 0;
                if ((((size_t)grow * G + gc) & 7) == 0) { /* 16-byte loads of 8 scales while whole ones remain */
                    for (; j + 8 <= nc; j += 8) {
                        const uint4 v = __ldg((const uint4 *)(srow + gc + j));
                        const uint16_t *e = (const uint16_t *)&v;
#pragma unroll
                        for (int q = 0; q < 8; ++q) sc_t[(j + q) * kTcRows + L] = e[q];
                    }
                }
#pragma unroll 8
                for (; j < nc; ++j) sc_t[j * kTcRows + L] = __ldg(srow + gc + j);
                for (int g = gc; g < gc + nc; ++g, ++gi) {
                    if (!ok) continue;
                    const float sc = bf16_bits_to_f32(sc_t[(g - gc) * kTcRows + L]);
                    const uint32_t db = gi % kTcAccBufs;
                    ok = tc_warp_wait(&sm->done[db], (gi / kTcAccBufs) & 1u, &sm->abort_flag, lane); /* tcgen05.ld is warp-wide: the warp goes on together or not at all */
                    if (!ok) {
                        if (lane == 0) tc_give_up(sm, P.status, ST_TC_D_FULL);
                        continue;
                    }
                    tc_fence_after();
                    if (L == 0) tc_stamp(P, 5, gi);
#pragma unroll
                    for (int t16 = 0; t16 < NT; ++t16) {
                        uint32_t d[16];
                        tmem_ld16(lane_addr + db * (uint32_t)NPAD + (uint32_t)(t16 * 16), d);
                        tmem_ld_wait();
#pragma unroll
                        for (int c = 0; c < 16; ++c) acc[t16 * 16 + c] = fmaf(sc, __uint_as_float(d[c]), acc[t16 * 16 + c]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm->d_empty[db]);
                    if (L == 0) tc_stamp(P, 6, gi);
                }
            }
            if (L == 0 && u == (int)blockIdx.x) tc_stamp(P, 7, 1);
            /* every epilogue thread passes the same barriers below whatever happened above */
            if (PAIRS) {
                /* SiLU(gate) * up, 16 tokens at a time: gate rows sit in lanes 0-63, up rows in lanes 64-127,
                 * so both halves hand their sums over through shared memory and ALL four warps then finish
                 * pairs - thread L takes pair L mod 64 and tokens 8 * (L / 64) .. + 7 of the batch. */
                const int pr = L & 63, half = L >> 6;
                const int p = t.row_a + pr; /* this rank's gate/up pair = column of the down projection */
                const int kb = p >> 6, piece = (p >> 3) & 7; /* K block of 64 columns of the down projection; 16-byte piece in it */
                uint8_t *tile = P.act_t + (size_t)kb * NPAD * 128 + tc_permute8(p & 7) * 2;
#pragma unroll
                for (int t16 = 0; t16 < NT; ++t16) {
                    float *mine = (L < 64 ? sm->ex_gate : sm->ex_up) + pr * 17;
#pragma unroll
                    for (int c = 0; c < 16; ++c) mine[c] = acc[t16 * 16 + c];
                    epi_bar();
                    if (ok) {
#pragma unroll
                        for (int c8 = 0; c8 < 8; ++c8) {
                            const int c = half * 8 + c8, m = t16 * 16 + c;
                            if (m < P.M) {
                                const uint16_t a = f32_to_bf16_bits(silu_mul(round_bf16(sm->ex_gate[pr * 17 + c]), round_bf16(sm->ex_up[pr * 17 + c])));
                                P.act[(size_t)m * P.N + p] = a;
                                *(uint16_t *)(tile + tc_tile_offset(m, piece)) = a;
                            }
                        }
                    }
                    epi_bar();
                }
            } else {
                bool finish = true;
                if (P.splits > 1) {
                    if (ok) {
#pragma unroll
                        for (int m = 0; m < NPAD; ++m)
                            if (m < P.M) __stcg(P.partial + ((size_t)t.sp * P.M + m) * P.N + grow, acc[m]);
                    }
                    __threadfence();
                    epi_bar();
                    if (L == 0) {
                        int last = 0;
                        if (!sm->abort_flag) {
                            const unsigned before = atomicAdd(P.arrivals + t.rb, 1u);
                            last = before == (unsigned)P.splits - 1u;
                            if (last) P.arrivals[t.rb] = 0u; /* ready for the next launch */
                        }
                        sm->last_arrival = last;
                    }
                    epi_bar();
                    finish = sm->last_arrival != 0;
                    epi_bar();
                    if (finish) {
                        /* the last of the row block's K splits to arrive adds them in split order */
                        __threadfence();
                        /* split by split, all tokens of a split together: the loads of one split are
                         * independent of one another, so they are in flight together (a loop of
                         * load-then-add per token serialises the trips to L2: 190 of them took 67 us) */
#pragma unroll
                        for (int m = 0; m < NPAD; ++m) acc[m] = 0.0f;
                        for (int q = 0; q < P.splits; ++q) {
                            const float *from = P.partial + (size_t)q * P.M * P.N + grow;
#pragma unroll
                            for (int m = 0; m < NPAD; ++m)
                                if (m < P.M) acc[m] += __ldcg(from + (size_t)m * P.N);
                        }
                    }
                }
                if (finish && ok) tc_down_output<NPAD>(P, sm, acc, grow, seq);
            }
            if (L == 0 && u == (int)blockIdx.x) tc_stamp(P, 7, 2);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kTcFirstMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, kTcTmemCols);
    }
}

/* x bf16 [M][K] -> tile order (see the head of this file); tokens M..npad-1 become zeros.  One thread
 * moves one run of 8 values. */
__global__ void tc_tile_input_kernel(uint8_t *__restrict__ xt, const uint16_t *__restrict__ x, int M, int npad, int K) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; /* = run * npad + n */
    const size_t total = (size_t)(K / 8) * npad;
    if (i >= total) return;
    const int n = (int)(i % npad);
    const size_t run = i / npad; /* g*16 + j: which run of 8 along K */
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (n < M) {
        const uint4 v = *(const uint4 *)(x + (size_t)n * K + run * 8);
        const uint16_t *e = (const uint16_t *)&v;
        uint16_t *d = (uint16_t *)&o;
#pragma unroll
        for (int k = 0; k < 8; ++k) d[((k & 3) << 1) | (k >> 2)] = e[k];
    }
    *(uint4 *)(xt + (run >> 3) * ((size_t)npad * 128) + tc_tile_offset(n, (int)(run & 7))) = o;
}

/* ---- host ----------------------------------------------------------------------------------- */
struct TcScratch {
    uint8_t *base = nullptr;
    size_t bytes = 0;
};
static TcScratch g_tc_scratch[64];
static std::mutex g_tc_mutex; /* guards the table; the scratch itself is shared by every call on the device */
static int g_tc_mode = 2; /* 0: always, 1: never, 2: where it measured faster than the mma.sync pair (tc_wanted) */

int tc_set_mode(int mode) {
    const int old = g_tc_mode;
    if (mode >= 0 && mode <= 2) g_tc_mode = mode;
    return old;
}
/* Measured on B200 (5120 x 17408, us per FFN, tcgen05 vs mma.sync pair): 8 tokens 79 vs 56, 16: 82 vs 73,
 * 24: 91 vs 93, 32: 93 vs 96, 48: 107 vs 177, 64: 123 vs 186; on TP=2 slices 32: 75 vs 77, 64: 114 vs 132.
 * So: more than 16 tokens, and enough gate/up units (intermediate size / 64) to occupy half the SMs -
 * smaller slices (TP=8 of that layer: 34 units) stay with the mma.sync pair. */
static bool tc_wanted(int tokens, int I, int sm_count) {
    return g_tc_mode == 0 || (g_tc_mode == 2 && tokens > 16 && 2 * (I / 64) >= sm_count);
}

/* The driver's tensor-map encoder, through the runtime (no link against the driver library). */
static PFN_cuTensorMapEncodeTiled_v12000 tc_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static bool tried = false;
    if (!tried) { /* callers hold g_tc_mutex */
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
        else
            (void)cudaGetLastError();
    }
    return fn;
}
/* packed rows [rows][K/2] as a 2-D byte tensor; a box is 128 bytes (two groups) of 64 rows, written to
 * shared memory with the 128-byte swizzle */
static int tc_weight_map(CUtensorMap *map, const void *w, int rows, int K) {
    PFN_cuTensorMapEncodeTiled_v12000 encode = tc_encoder();
    if (!encode) return fail(FFN_ERR_CUDA, "tcgen05 FFN: the driver offers no cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
    const cuuint32_t box[2] = {(cuuint32_t)kTcRowPitch, (cuuint32_t)kTcBoxRows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(w), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FFN_ERR_CUDA, "tcgen05 FFN: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return FFN_OK;
}

static int tc_tiles_for(int tokens) { return (tokens + 15) / 16; }
static int tc_stage_bytes(int nt) { return kTcRows * kTcRowPitch + kTcGroupsPerStage * nt * 16 * 256; }
static int tc_smem_bytes(int nt, int stages) { return kTcHeader + kTcScaleBytes + stages * tc_stage_bytes(nt); }
/* Depth of the packed ring for `nt` 16-token column blocks: whatever shared memory holds, at most 8.
 * The ring has to cover the latency of a TMA load (about 1.5 us under load) at the SM's share of the
 * HBM rate, i.e. some 70 KB of packed rows in flight. */
static bool tc_depth(int nt, int smem_optin, int *stages) {
    int n = (smem_optin - kTcHeader - kTcScaleBytes) / tc_stage_bytes(nt);
    if (n > kTcMaxStages) n = kTcMaxStages;
    *stages = n;
    return n >= 2;
}
static int tc_splits(int H, int I, int sm_count) {
    const int blocks = H / kTcRows, G = I / FFN_INT4_GROUP;
    int sp = sm_count / blocks;
    if (sp > kTcMaxSplits) sp = kTcMaxSplits;
    if (sp > G / 2) sp = G / 2;
    return sp < 1 ? 1 : sp;
}
static bool tc_admits(int tokens, int H, int I, int sm_count, int smem_optin) {
    if (tokens < 1 || tokens > 64 || H <= 0 || I <= 0) return false;
    if (H % kTcRows || I % 64 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP) return false;
    int stages;
    return tc_depth(tc_tiles_for(tokens), smem_optin, &stages) && sm_count >= 1;
}

bool tc_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes) {
    if (!tc_wanted(tokens, I, sm_count) || !tc_admits(tokens, H, I, sm_count, smem_optin)) return false;
    const int nt = tc_tiles_for(tokens), sp = tc_splits(H, I, sm_count);
    int stages = 0;
    tc_depth(nt, smem_optin, &stages);
    snprintf(out, out_bytes,
             "kernel=tcgen05_pair token_columns=%d threads=%d smem=%d stages=%d operand_buffers=%d accumulator_buffers=%d "
             "tmem_columns=%d gate_up_units=%d gate_up_ctas=%d down_units=%d down_k_splits=%d",
             nt * 16, kTcThreads, tc_smem_bytes(nt, stages), stages, kTcABufs, kTcAccBufs, kTcTmemCols, I / 64,
             I / 64 < sm_count ? I / 64 : sm_count, (H / kTcRows) * sp, sp);
    return true;
}

template <int NT>
static int tc_launch_pair(const TcParams &A, const TcParams &B, int sm_count, cudaStream_t stream) {
    const int smem = tc_smem_bytes(NT, A.stages);
    FFN_CUDA_TRY(cudaFuncSetAttribute(ffn_tc_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "tcgen05 gate/up: shared-memory opt-in");
    FFN_CUDA_TRY(cudaFuncSetAttribute(ffn_tc_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "tcgen05 down: shared-memory opt-in");
    ffn_tc_kernel<NT, true><<<A.units < sm_count ? A.units : sm_count, kTcThreads, smem, stream>>>(A);
    FFN_CUDA_TRY(cudaGetLastError(), "tcgen05 gate/up launch");
    ffn_tc_kernel<NT, false><<<B.units < sm_count ? B.units : sm_count, kTcThreads, smem, stream>>>(B);
    FFN_CUDA_TRY(cudaGetLastError(), "tcgen05 down launch");
    return FFN_OK;
}

/* The arrival counters of the down launch are zero between launches; a launch that gave up may leave
 * some behind, so clearing the device's status also clears them. */
void tc_reset_sync() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
    std::lock_guard<std::mutex> lock(g_tc_mutex);
    if (g_tc_scratch[dev].base) (void)cudaMemset(g_tc_scratch[dev].base, 0, 4096);
}

/* normed bf16 [tokens][H] -> layer_out bf16 [tokens][H]; `act` receives act in natural order. */
int tc_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                  const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual, unsigned *status) {
    int dev = 0, smem_optin = 0, sm_count = 0;
    FFN_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(FFN_ERR_CONFIG, "device index %d out of range", dev);
    FFN_CUDA_TRY(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "smem opt-in");
    FFN_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev), "SM count");
    if (!tc_wanted(tokens, I, sm_count) || !tc_admits(tokens, H, I, sm_count, smem_optin)) return FFN_NOT_ADMITTED;
    if (((uintptr_t)w->gate_up_i4 & 15) || ((uintptr_t)w->down_i4 & 15) || ((uintptr_t)normed & 15)) return FFN_NOT_ADMITTED;
    if (((uintptr_t)w->gate_up_i4_scales & 15) || ((uintptr_t)w->down_i4_scales & 15)) return FFN_NOT_ADMITTED;
    const size_t counters = 4096;
    if ((size_t)(H / kTcRows) * sizeof(unsigned) > counters) return FFN_NOT_ADMITTED;
    /* layout: [arrival counters 4 KiB | input in tile order | act in tile order | partial sums], sized for 64 tokens */
    const size_t xt_bytes = ((size_t)64 * H * 2 + 255) / 256 * 256, at_bytes = ((size_t)64 * I * 2 + 255) / 256 * 256;
    const size_t want = counters + xt_bytes + at_bytes + (size_t)kTcMaxSplits * 64 * H * sizeof(float);
    std::lock_guard<std::mutex> lock(g_tc_mutex);
    TcScratch &sc = g_tc_scratch[dev];
    if (sc.bytes < want) {
        if (sc.base) { FFN_CUDA_TRY(cudaDeviceSynchronize(), "tcgen05 FFN: scratch regrow"); cudaFree(sc.base); }
        sc.base = nullptr; sc.bytes = 0;
        if (cudaMalloc(&sc.base, want) != cudaSuccess) { (void)cudaGetLastError(); return fail(FFN_ERR_ALLOC, "tcgen05 FFN: cannot allocate %zu bytes of scratch", want); }
        FFN_CUDA_TRY(cudaMemset(sc.base, 0, want), "tcgen05 FFN: clear scratch");
        sc.bytes = want;
    }
    const int nt = tc_tiles_for(tokens), npad = nt * 16;
    uint8_t *xt = sc.base + counters, *act_t = xt + xt_bytes;
    const size_t runs = (size_t)(H / 8) * npad;
    tc_tile_input_kernel<<<(unsigned)((runs + 255) / 256), 256, 0, stream>>>(xt, (const uint16_t *)normed, tokens, npad, H);
    FFN_CUDA_TRY(cudaGetLastError(), "tile-order input launch");

    TcParams A = {};
    int st = tc_weight_map(&A.wmap, w->gate_up_i4, 2 * I, H);
    if (st) return st;
    A.xt = xt; A.s = (const uint16_t *)w->gate_up_i4_scales;
    A.M = tokens; A.npad = npad; A.N = I; A.K = H; A.up_offset = I;
    A.units = I / 64; A.splits = 1;
    tc_depth(nt, smem_optin, &A.stages);
    A.act = (uint16_t *)act; A.act_t = act_t;
    A.tp = 1; A.status = status; A.trace = fused_get_trace();
    TcParams B = {};
    if ((st = tc_weight_map(&B.wmap, w->down_i4, H, I))) return st;
    B.xt = act_t; B.s = (const uint16_t *)w->down_i4_scales;
    B.M = tokens; B.npad = npad; B.N = H; B.K = I;
    B.splits = tc_splits(H, I, sm_count); B.units = (H / kTcRows) * B.splits;
    B.stages = A.stages;
    B.out = (uint16_t *)layer_out; B.residual = (uint16_t *)residual;
    B.partial = (float *)(sc.base + counters + xt_bytes + at_bytes); B.arrivals = (unsigned *)sc.base;
    B.tp = 1; B.status = status; B.trace = A.trace ? A.trace + 512 : nullptr;
    if (tp && tp->tp > 1) {
        if (tokens * H > tp->slot_stride) return fail(FFN_ERR_CONFIG, "tcgen05 FFN: %d tokens exceed the exchange buffer", tokens);
        A.tp_seq = tp->seq;
        B.tp = tp->tp; B.rank = tp->rank; B.slot_stride = tp->slot_stride;
        B.peer_slots = tp->peer_slots; B.tp_seq = tp->seq;
    }
    switch (nt) {
        case 1: return tc_launch_pair<1>(A, B, sm_count, stream);
        case 2: return tc_launch_pair<2>(A, B, sm_count, stream);
        case 3: return tc_launch_pair<3>(A, B, sm_count, stream);
        default: return tc_launch_pair<4>(A, B, sm_count, stream);
    }
}

/* Byte offset of activation (token, k) in the tile order the tcgen05 pair reads (host arithmetic: the
 * layout's definition for tests and for an engine that wants to write activations that way itself). */
long long tc_tile_order_offset(int token, int k, int npad) {
    const int block = k >> 6, piece = (k >> 3) & 7, e = k & 7;
    return (long long)block * npad * 128 + tc_tile_offset(token, piece) + (((e & 3) << 1) | (e >> 2)) * 2;
}

/* 3..64 tokens: the tcgen05 pair where it takes the shape, else the mma.sync pair. */
int batched_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                       const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual, unsigned *status) {
    const int st = tc_ffn_launch(stream, normed, act, layer_out, w, tokens, H, I, tp, residual, status);
    if (st != FFN_NOT_ADMITTED) return st;
    return mma_ffn_launch(stream, normed, act, layer_out, w, tokens, H, I, tp, residual, status);
}

}  // namespace ffn
