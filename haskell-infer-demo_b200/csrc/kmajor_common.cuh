/*
 * kmajor_common.cuh - pieces shared by the two decode kernels that work over k-major copies of the
 * down projection (ffn_kmajor.cu: dp4a consumers; ffn_imma.cu: int8 tensor-core consumers): the
 * contiguous work partition, the tagged 8-byte words that carry partial sums and the residual stream
 * between CTAs and layers without fences, the relaxed arrival counters used as polling hints, and the
 * host-side view of the per-device hand-over buffers and of the registered k-major copies.
 */
#pragma once

#include "stream_common.cuh"

namespace ffn {

/* first k-block of CTA `cta` (total * ctas < 2^32 is checked on the host) */
__device__ __forceinline__ int km_begin(int total, int cta, int ctas) {
    return (int)(((unsigned)total * (unsigned)cta) / (unsigned)ctas);
}

/* Words between two CTAs' partial sums: the tokens' rows plus 48 words of padding, so that the words of
 * one output row (one per CTA, which a reducer reads together) do not sit a multiple of 4 KB apart. */
__host__ __device__ __forceinline__ size_t km_partial_stride(int tokens, int hidden) { return (size_t)tokens * hidden + 48; }

/* Tag of the words layer number `e` (counted per device since start-up) leaves inside its GPU: never
 * zero (zero marks a word nobody has written), and two consecutive layers never share one, also when
 * the 32-bit count wraps. */
__device__ __forceinline__ unsigned km_tag(unsigned e) { return e | 0x80000000u; }

/* tagged words inside one GPU: {FP32 value, tag} as one 8-byte store / load */
__device__ __forceinline__ unsigned long long km_word(float v, unsigned tag) {
    return ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
}
/* Plain stores that go to the L2 (.cg): stores qualified .relaxed.gpu measured a full L2 round trip
 * each, one after the other (40 stores = 12 us); the readers accept a word on its tag only, so no
 * ordering between the stores is needed. */
__device__ __forceinline__ void km_store2(unsigned long long *p, unsigned long long a, unsigned long long b) { /* 16-byte aligned */
    asm volatile("st.global.cg.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void km_store1(unsigned long long *p, unsigned long long a) {
    asm volatile("st.global.cg.u64 [%0], %1;" ::"l"(p), "l"(a) : "memory");
}
/* Loads of tagged words come in batches (up to 20 per lane) whose results are all checked afterwards,
 * so they must overlap: plain loads served by the L2 (.cg: no L1 allocation, so a repeated poll reads
 * the L2 again).  Loads qualified .relaxed.gpu measured one L2 round trip EACH, back to back - 6 us for
 * a batch.  A word is only ever accepted on its tag, so a stale answer costs a retry, never an error. */
__device__ __forceinline__ unsigned long long km_load1(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.global.cg.u64 %0, [%1];" : "=l"(w) : "l"(p));
    return w;
}
__device__ __forceinline__ void km_load2(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.global.cg.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p));
}
__device__ __forceinline__ unsigned km_load_counter(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void km_arrive_counter(unsigned *p) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ uint2 km_lds8(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

/* A relaxed counter as a HINT that polling the tagged words is worth starting: waits (bounded) until
 * it has reached `target`.  Correctness never depends on it - the words validate themselves. */
__device__ __forceinline__ bool km_wait_counter(const unsigned *p, unsigned target, volatile int *abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if ((int)(km_load_counter(p) - target) >= 0) return true;
        if ((i & 63) == 63 && *abort_flag) return false;
        __nanosleep(40);
    }
    return false;
}

/* ---- host side (ffn_kmajor.cu) ------------------------------------------------------------- */
struct KmDeviceView {
    int sm_count, smem_optin, cooperative;
    unsigned *sync;              /* [0] arrivals "partials stored", [1] arrivals "h published", [2] the counters' value at
                                    the start of the launch, [3] layers run so far (base of the tags) */
    unsigned long long *partial; /* [sm_count][2 or 4 tokens][hidden] tagged words */
    unsigned long long *hx;      /* [tokens][hidden] tagged words */
};
/* Per-device buffers sized for `hidden` and `tokens` (allocated or regrown on first use). */
int kmajor_device_view(int hidden, int tokens, KmDeviceView *out);
/* The registered k-major copy of the down projection at device address `down_i4`, if it has this shape
 * and lives on device `dev`. */
bool kmajor_lookup(const void *down_i4, int hidden, int inter, int dev, const uint32_t **wt, const uint16_t **st);

}  // namespace ffn
