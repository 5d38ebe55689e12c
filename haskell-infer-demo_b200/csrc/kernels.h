/* kernels.h - internal (C++) interface between the kernel translation units and the C ABI. */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ffn_int4.h"

namespace ffn {

/* basic_kernels.cu */
int gemm_int4_generic(const void *a, const void *packed, const void *scales, void *out_bf16,
                      float *out_f32, int M, int N, int K, cudaStream_t stream);
int silu_mul_packed(void *out, const void *packed, int tokens, int inter, cudaStream_t stream);
int gemma_rms_norm(void *out, const void *x, const void *w, int cols, int rows, float eps, int gemma,
                   cudaStream_t stream);
int residual_add(void *dst, const void *src, int n, cudaStream_t stream);
int residual_norm(void *normed, void *residual, const void *sublayer, const void *w, int cols, int rows, float eps,
                  int gemma, cudaStream_t stream);
int silu_mul_pair(void *out, const void *gate, int n, cudaStream_t stream);
/* Launch geometry as text, computed from the shape alone (no device needed); false = the kernel does not take the shape. */
bool fused_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes);
bool mma_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes);
int dequantize_int4(void *out, const void *packed, const void *scales, int N, int K, int *bad,
                    cudaStream_t stream);

/* ffn_fused.cu */
#define FFN_NOT_ADMITTED 1 /* internal: the fused kernel does not take this shape */
/* M-dispatching GEMM: one or two activation rows go through the streaming kernel's single-matrix
 * mode (when the shape and the alignment allow), everything else through the generic kernel. */
int gemm_int4_dispatch(const void *a, const void *packed, const void *scales, void *out, int M, int N,
                       int K, cudaStream_t stream);
/* The single-launch fused FFN (gate/up + SiLU*up + down).  Returns FFN_NOT_ADMITTED when the shape
 * is outside what it supports, so the caller can take the three-kernel route. */
int fused_ffn_try(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                  const FfnMlpWeights *w, int tokens, int H, int I);

/* Layout of one rank's exchange buffer:
 *   [ call counter u32, pad to kTpHeaderBytes | slots: [2][tp][max_tokens * hidden] x 8 bytes ]
 * A slot element is ONE 8-byte word {FP32 partial sum, call number + 1}: the sender writes it with a
 * single store into every rank's buffer and the receiver polls the word itself until the tag is the
 * current call's.  Value and "it has arrived" travel in the same transaction, so the exchange needs
 * no fence, no separate flag and no second trip over NVLink, and the test does not depend on which
 * kernel served the earlier calls (the single-pass and the batched kernels may alternate freely on
 * one communicator).  Buffers alternate by call parity: a rank can be at most one call ahead of a
 * peer, because completing a call needs every peer's words of that call. */
constexpr int kTpMaxRanks = 16;
constexpr size_t kTpSeqOffset = 0;
constexpr size_t kTpHeaderBytes = 256;
constexpr uint32_t kTpPollLimit = 1u << 20; /* polls of one tagged word before a receiver gives up (about a second) */

/* The tag the exchange words of call number `seq` carry.  Never zero (zero marks a word nobody has
 * written since the buffer was cleared), also when the 32-bit call counter wraps. */
__host__ __device__ __forceinline__ unsigned tp_tag(unsigned seq) { return seq % 0xFFFFFFFFu + 1u; }

/* A plain 8-byte store (one transaction, posted over NVLink): a store qualified .relaxed.sys is
 * completed before the thread's next strong access issues - measured as one full round trip per
 * store inside a GPU - which would put a link round trip in front of every following store and of
 * the first poll.  The receiver accepts a word on its tag only, so nothing else has to be ordered. */
__device__ __forceinline__ void tp_store_tagged(unsigned long long *p, float v, unsigned tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.global.cg.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
/* true when the word carries `tag`; *v is its value then */
__device__ __forceinline__ bool tp_load_tagged(const unsigned long long *p, unsigned tag, float *v) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    *v = __uint_as_float((unsigned)w);
    return (unsigned)(w >> 32) == tag;
}

/* Waits (bounded) until the `tp` words first[r * stride] all carry `tag`, then returns their values added
 * in rank order.  All loads of a round are issued before any tag is looked at, so they overlap (plain
 * loads served by the L2, where writes arriving over NVLink land; a load qualified .relaxed.sys is
 * completed before the next one issues, which made eight ranks cost eight round trips). */
__device__ __forceinline__ bool tp_wait_sum(const unsigned long long *first, size_t stride, int tp, unsigned tag,
                                            const volatile int *abort_flag, uint32_t sleep_ns, float *sum) {
    unsigned long long w[kTpMaxRanks];
    bool in = false;
    for (uint32_t k = 0; k < kTpPollLimit && !in; ++k) {
        in = true;
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; ++r) {
            w[r] = (unsigned long long)tag << 32;
            if (r < tp) asm volatile("ld.global.cg.u64 %0, [%1];" : "=l"(w[r]) : "l"(first + (size_t)r * stride));
        }
#pragma unroll
        for (int r = 0; r < kTpMaxRanks; ++r) in = in && (unsigned)(w[r] >> 32) == tag;
        if (!in) {
            if ((k & 1023u) == 1023u && abort_flag && *abort_flag) break;
            __nanosleep(sleep_ns);
        }
    }
    float a = 0.0f;
#pragma unroll
    for (int r = 0; r < kTpMaxRanks; ++r)
        if (r < tp) a += __uint_as_float((unsigned)w[r]);
    *sum = a;
    return in;
}

/* Tensor-parallel exchange tables (device arrays of per-rank pointers, set up once at load). */
struct FusedTp {
    int tp, rank;
    unsigned long long *const *peer_slots; /* [tp] -> each rank's [2][tp][slot_stride] tagged words */
    int slot_stride;             /* elements per (parity, rank) slot */
    unsigned *seq;               /* this rank's call counter for this communicator (device word) */
};
/* Optional RMSNorm fused into the kernel's input stage (weight == NULL: the input is already normalized). */
struct FusedNorm {
    const void *weight; /* bf16 [H] */
    float eps;
    int gemma;          /* 1: scale by (1 + w), 0: by w */
};
int fused_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                     const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual,
                     const FusedNorm *norm);
/* Reads (synchronously) the status word the fused kernel writes when a bounded wait runs out:
 * 0 = fine, else (where | cta << 8).  With reset, a non-zero status also clears the kernel's
 * synchronisation words so the next launch starts clean. */
int fused_status(unsigned *status_out, bool reset);
/* The same for the status word inside the static scratch array of the allocation-free entry point. */
int fused_status_noalloc(unsigned *status_out, bool reset);
bool fused_noalloc_in_use();
bool gemv_describe_plan(int tokens, int N, int K, int sm_count, int smem_optin, char *out, size_t out_bytes);
void fused_set_trace(long long *device_buffer);
long long *fused_get_trace();
/* ffn_kmajor.cu: the persistent multi-layer kernel over k-major copies of the down projections
 * (registered per layer with ffn_decode_layer_prepare).  `layers` are `num_layers` consecutive layers
 * of one stack (1 for a single FFN call); with_norm fuses each layer's RMSNorm (post_norm_w) into its
 * input stage.  FFN_NOT_ADMITTED when a layer is not registered or the shape is outside the kernel. */
int kmajor_ffn_launch(cudaStream_t stream, const void *x, void *act, void *layer_out, const FfnMlpWeights *layers,
                      int num_layers, int tokens, int H, int I, const FusedTp *tp, void *residual, int with_norm,
                      float eps, int gemma, unsigned *status);
void kmajor_reset_sync();
int fused_set_launch_overlap(int on); /* ffn_fused.cu: programmatic dependent launch on or off; returns the previous setting */
/* ffn_imma.cu: the same contract for 1..4 tokens with the inner products on the INT8 tensor cores.
 * kmajor_ffn_launch tries it first only after kmajor_prefer_dp4a(0) (A/B measurements, tests): it measured
 * slower than the dp4a kernel, which is the default. */
int imma_ffn_launch(cudaStream_t stream, const void *x, void *act, void *layer_out, const FfnMlpWeights *layers,
                    int num_layers, int tokens, int H, int I, const FusedTp *tp, void *residual, int with_norm,
                    float eps, int gemma, unsigned *status);
bool imma_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes);
int kmajor_prefer_dp4a(int on); /* returns the previous setting */
bool kmajor_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes);
/* ffn_mma.cu: the tensor-core path for 3..64 tokens (two launches: gate/up + SiLU*up, down + reduce). */
/* ffn_tc.cu: the same contract on tcgen05 tensor cores (accumulators in tensor memory); batched_ffn_launch
 * tries it first and falls back to the mma.sync pair for shapes it does not take.  tc_set_mode: 0 always,
 * 1 never, 2 (default) where it measured faster (more than 16 tokens, gate/up units for half the SMs);
 * returns the previous mode. */
int tc_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                  const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual, unsigned *status);
int batched_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                       const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual, unsigned *status);
bool tc_describe_plan(int tokens, int H, int I, int sm_count, int smem_optin, char *out, size_t out_bytes);
int tc_set_mode(int mode);
long long tc_tile_order_offset(int token, int k, int npad);
void tc_reset_sync();
int mma_ffn_launch(cudaStream_t stream, const void *normed, void *act, void *layer_out,
                   const FfnMlpWeights *w, int tokens, int H, int I, const FusedTp *tp, void *residual, unsigned *status);
/* Device address of the status word shared by the kernels of this library (allocating it on first use). */
int fused_status_word(unsigned **out);
/* The fused FFN with its scratch in a static device array: calls no allocating routine. */
int fused_ffn_launch_noalloc(cudaStream_t stream, const void *normed, void *layer_out,
                             const FfnMlpWeights *w, int tokens, int H, int I);

}  // namespace ffn
