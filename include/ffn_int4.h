/*
 * ffn_int4.h - C ABI of libffn_int4.so: the weight-only INT4 (symmetric, group 128, BF16 scales)
 * dense-FFN decode path for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only.  Every entry point returns FFN_OK (0) or a negative status and
 * leaves a message in ffn_int4_last_error() (thread-local, valid until the next call on the
 * thread) - the convention of the reference engine ABI (csrc/include/engine.h:264-276).  No C++
 * exception crosses this boundary.  All device pointers belong to the CUDA device that is current
 * on the calling thread; `stream` arguments are `cudaStream_t` passed as `void *` (NULL = the
 * default stream).  There is no CPU fallback: without a usable CUDA device every compute entry
 * point fails with FFN_ERR_CUDA.
 *
 * Concurrency: the FFN entry points of one device (ffn_forward_mlp*, ffn_forward_mlp_tp,
 * ffn_decode_stack, ffn_gemm_int4_bf16 with one or two rows, ffn_tp_allreduce_sum) share that
 * device's synchronisation words, kernel status word and, for 3..64 tokens, one scratch region
 * (permuted activations, split-K partial sums, arrival counters).  Calls on one device must
 * therefore be serialised: issue them on one stream, or order the streams with events.  Calls on
 * different devices are independent.  The first call on a device, and the first call of the batched
 * path there, allocate these words with cudaMalloc: make them before capturing a CUDA graph.
 *
 * Data layouts (identical to the reference's, csrc/include/linear_weight.h:12-13, 46-54):
 *   packed [N][K/2]   u8, row-major; byte j of a row = code(k=2j) | code(k=2j+1) << 4; codes are
 *                     4-bit two's complement in [-7, 7]; 0x8 is the reserved invalid code
 *   scales [N][K/128] bf16, row-major (row, group)
 *   gate/up pair      [2*I_local][H]: the rank's gate rows, then its up rows
 *   down              [H][I_local]
 *   activations       bf16 [M][H]; outputs bf16 [M][H]
 */
#ifndef FFN_INT4_H
#define FFN_INT4_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FFN_INT4_ABI_VERSION 1
#define FFN_INT4_GROUP 128

/* Status codes: the values of ENGINE_OK / ENGINE_ERR_* (csrc/include/engine.h:264-270). */
#define FFN_OK 0
#define FFN_ERR_CUDA (-1)    /* CUDA runtime error, or a bounded device-side wait ran out */
#define FFN_ERR_ALLOC (-2)   /* device or host allocation failed */
#define FFN_ERR_WEIGHTS (-3) /* artifact / manifest refused */
#define FFN_ERR_CONFIG (-4)  /* invalid argument or unsupported shape */
#define FFN_ERR_STATE (-5)   /* call order or object state */

/* Replaces engine_last_error (csrc/include/engine.h:272-276) for this library's calls. */
const char *ffn_int4_last_error(void);
int ffn_int4_abi_version(void);

/* Synchronises the current device and reports whether any fused kernel since the last call gave
 * up on a bounded wait (every device-side wait in this library has an iteration limit; on expiry
 * the kernel records where and returns instead of hanging).  Returns FFN_OK, or FFN_ERR_CUDA with
 * `where` (1..8) and `cta` filled; a non-zero status is cleared and the kernel's synchronisation
 * words are reset, the analogue of the reference's "failed forward needs engine_reset"
 * (csrc/engine.cu:1723-1730).  No counterpart function in the reference. */
int ffn_int4_device_status(int *where, int *cta);

/* The same report for ffn_forward_mlp_prepared_noalloc, whose kernel keeps its status word inside
 * the library's static scratch array: synchronises the current device, copies the word to the host
 * and, when it is non-zero, clears it together with the array's synchronisation words.  Calls no
 * allocating routine, so a host that cannot allocate can use it (ffn_int4_device_status allocates
 * the regular path's words on first use; it also reports this word once the array is in use on the
 * device).  A wait that ran out stays on record across later calls until one of the two functions
 * reads it.  No counterpart in the reference. */
int ffn_int4_noalloc_status(int *where, int *cta);

/* The identity of this library's arithmetic for the reference's execution manifest: the members it
 * contributes to the `numerical_policy` fields (csrc/manifest.c:385-434), as text of the form
 * "key":"value","key":"value" with sorted keys.  `weight_quantization` carries the reference's own
 * value for INT4 operands (csrc/manifest.c:433-434, set at csrc/engine.cu:1357); the other members
 * name the accumulation scheme, the rounding points and the cross-rank reduction, so that
 * numerical_policy_id moves when the engine is linked against this library and semantic_id /
 * deployment_id do not (the property tests/manifest_test.c:335-352 checks for the INT4 switch). */
const char *ffn_int4_numerical_policy(void);

/* Which kernel a call of this shape takes and its launch geometry (grid, shared memory, pipeline
 * stages, tile sizes, K splits), as one line of key=value text, for a device with `sm_count` SMs and
 * `smem_optin` bytes of opt-in shared memory per block.  Pure host arithmetic: needs no GPU, so the
 * planning can be checked for any shape anywhere.  `intermediate` is the rank-local size.  No
 * counterpart in the reference (its launch shapes are fixed constants, csrc/kernels/gemm_quant.cu:20-31). */
int ffn_int4_describe_plan(int tokens, int hidden, int intermediate, int sm_count, int smem_optin, char *out,
                           size_t out_bytes);
/* The same for one ffn_gemm_int4_bf16 call of m rows against an [n][k] matrix. */
int ffn_int4_describe_gemm_plan(int m, int n, int k, int sm_count, int smem_optin, char *out, size_t out_bytes);

/* Debugging aid: when given a device buffer of 16 int64 per SM (16 x 148 on B200), every CTA of every
 * later decode-kernel launch writes global-timer stamps (ns) of its pipeline events to its own 16
 * words; the tcgen05 pair instead has CTA 0 write SM-clock stamps of its roles' first 64 groups to words
 * [role * 64 + group] (gate/up launch) and [512 + role * 64 + group] (down launch).  NULL switches it off.  No counterpart in the
 * reference (its profiler times whole regions with events, csrc/profile.cu:114-144). */
void ffn_int4_debug_trace(void *device_buffer);

/* Chooses between the single-launch fused FFN kernel (default, 1) and the three-kernel route
 * (gate/up GEMM, SiLU*up, down GEMM - the reference's launch structure, csrc/kernels/layers.cu:
 * 127-145) for ffn_forward_mlp*.  Both are CUDA paths; the switch exists for A/B measurement.
 * Returns the previous setting. */
int ffn_int4_set_fused(int enabled);

/* ------------------------------------------------------------------------------------------- */
/* Operator level                                                                              */
/* ------------------------------------------------------------------------------------------- */

/* Replaces gemm_int4_bf16 (csrc/include/layers.h:376-377; csrc/kernels/gemm_quant.cu:204-254).
 * out[M][N] (bf16) = a[M][K] (bf16) x dequant(packed, scales)[N][K]^T, FP32 accumulation, one
 * BF16 rounding.  Same refusals as the reference, returned as FFN_ERR_CONFIG instead of thrown:
 * negative extent, K <= 0, group <= 0, null buffer, K not a whole number of groups; this
 * library additionally requires group == 128 (the only group the format defines,
 * csrc/linear_weight.cpp:63-68).  M == 0 or N == 0 is a successful no-op.  Asynchronous on
 * `stream`.  One or two rows (the decode case: the FFN's matrices on their own, attention / GDN
 * projections, the LM head) stream through the persistent bulk-copy kernel when N % 8 == 0, K <=
 * 34816 (17408 for two rows) and the three operands are 16-byte aligned; everything else takes the
 * shape-generic kernel.  A non-finite activation makes the outputs it reaches non-finite in both. */
int ffn_gemm_int4_bf16(const void *a, const void *packed, const void *scales, void *out, int M,
                       int N, int K, int group, void *stream);

/* Replaces kernel_silu_mul_packed (csrc/kernels/silu.cu:76-95): out[t][i] =
 * bf16(silu(packed[t][i]) * packed[t][I + i]); packed is bf16 [tokens][2I]. */
int ffn_silu_mul_packed(void *out, const void *packed, int tokens, int intermediate, void *stream);

/* Replaces kernel_gemma_rms_norm (csrc/kernels/flashinfer_norm.cu:22-44): out = bf16(x *
 * rsqrt(mean(x^2) + eps) * (1 + w)) per row, FP32 arithmetic. */
int ffn_gemma_rms_norm(void *out, const void *x, const void *weight, int cols, int rows, float eps,
                       void *stream);

/* Replaces kernel_residual_norm (csrc/kernels/flashinfer_norm.cu:112-174; decl csrc/include/kernels.h): the
 * residual update and the norm that follows it in one pass.  residual <- bf16(f32(residual) +
 * f32(sublayer)) is stored, and normed = bf16(r * rsqrt(mean(r^2) + eps) * (weight + (gemma ? 1 : 0)))
 * is computed from the ROUNDED r, as the reference's rounding rule requires.  All bf16 [rows][hidden]
 * (weight [hidden]); same refusals ("invalid shape or epsilon", "null buffer") as status codes. */
int ffn_residual_norm(void *normed, void *residual, const void *sublayer, const void *weight, int hidden, int rows,
                      float eps, int gemma, void *stream);

/* Replaces kernel_silu_mul (csrc/kernels/silu.cu:29-52): out[i] = bf16(silu(gate[i]) * gate[n + i]) over a
 * contiguous [gate[n] | up[n]] bf16 buffer; same refusals (negative n; n >= 8 needs n % 8 == 0 and
 * 16-byte aligned buffers). */
int ffn_silu_mul(void *out, const void *gate, int n, void *stream);

/* Replaces kernel_residual_add (csrc/kernels/gdn_norm.cu:121-136): dst = bf16(f32(dst)+f32(src)). */
int ffn_residual_add(void *dst, const void *src, int n, void *stream);

/* Replaces linear_quantize_int4 (csrc/include/linear_weight.h; csrc/linear_weight.cpp:108-176), which the
 * reference's offline converter reaches once per tensor through a subprocess
 * (scripts/quantize_weights.py:136-156), for weights that are in device memory: FP32 [n][k] ->
 * packed [n][k/2] and BF16 scales [n][k/128], byte-identical to the reference's output (group
 * maximum, scale = BF16_RNE(max/7) with 1.0 for an all-zero group, q = clip(nearbyint(w/scale),
 * -7, 7) against the rounded scale, low K index in the low nibble).  Same refusals, reported before
 * anything is written: k % 128, n % 8 (FFN_ERR_CONFIG); a non-finite element, or a group whose scale
 * does not round to a positive finite BF16 (FFN_ERR_WEIGHTS, the message names the element or the
 * row and group).  Synchronises `stream` (the refusals need the checking pass's answer). */
int ffn_quantize_int4(const void *weights, void *packed, void *scales, long long n, long long k, void *stream);

/* Writes float(code) * float(scale) for every element of a packed [N][K] weight to out (FP32
 * [N][K]), so that the "dequantized weights are bit-exact" bar can be checked against
 * linear_dequantize_int4 (csrc/linear_weight.cpp:178-216).  It uses the shape-generic kernel's
 * unpack routine; the streaming and the tensor-core kernels widen the codes in their own ways, which
 * the tests pin separately with one-hot activations (a single non-zero activation makes their
 * arithmetic exact, so their outputs must then equal code * scale * activation bit for bit).
 * `bad` (device int, may be NULL) receives the number of reserved 0x8 nibbles met. */
int ffn_dequantize_int4(void *out, const void *packed, const void *scales, int N, int K, int *bad,
                        void *stream);

/* Field-for-field mirror of the reference's MlpWeights (csrc/include/layers.h:54-70), so the
 * engine's own struct can be passed unchanged.  Only the INT4 members and post_norm_w are read. */
typedef struct {
    const void *gate_proj_w;
    const void *up_proj_w;
    const void *down_proj_w;
    const void *post_norm_w;       /* bf16 [H], raw Gemma weight; NULL skips the norm */
    const uint8_t *gate_up_i4;     /* [2I][H/2] */
    const void *gate_up_i4_scales; /* bf16 [2I][H/128] */
    const uint8_t *down_i4;        /* [H][I/2] */
    const void *down_i4_scales;    /* bf16 [H][I/128] */
    int i4_group;
} FfnMlpWeights;

/* Field-for-field mirror of the reference's ModelDims (csrc/include/layers.h:19-47).  Read:
 * hidden_size, intermediate_size (the rank-local one), norm_style (0 = Gemma), rms_eps,
 * max_chunk. */
typedef struct {
    int hidden_size;
    int intermediate_size;
    int num_heads;
    int num_kv_heads;
    int head_dim;
    int rotary_dim;
    int norm_style;
    int attn_output_gate;
    int q_gate_interleave;
    int num_layers;
    int vocab_size;
    float rms_eps;
    float rope_theta;
    int max_seq_len;
    int gdn_conv_dim;
    int gdn_value_dim;
    int gdn_num_v_heads;
    int gdn_num_k_heads;
    int gdn_head_dim;
    int gdn_conv_kernel;
    int mla_kv_lora_rank;
    int mla_qk_nope_head_dim;
    int mla_qk_rope_head_dim;
    int mla_v_head_dim;
    int max_chunk;
} FfnModelDims;

/* Replaces forward_mlp (csrc/include/layers.h:335-337; csrc/kernels/layers.cu:149-160) for the
 * INT4 operands: post-norm (when post_norm_w is set) -> gate/up -> SiLU*up -> down, written to
 * layer_out [tokens][H] as BF16 with the reference's three rounding points.  `cublas` is
 * accepted and ignored (no cuBLAS on this path).  `ws` is the reference's workspace
 * (tokens*(H+3I) bf16, csrc/kernels/layers.cu:65, 117-118); the normalized activation is left
 * in ws[0 .. tokens*H) as the reference leaves it, and the activation a in its usual slot.  Unlike the reference
 * (csrc/kernels/layers.cu:126) every token count in [1, max_chunk] takes the INT4 path; a
 * weight set without INT4 operands is refused with FFN_ERR_CONFIG (there is no BF16 path here). */
int ffn_forward_mlp(void *cublas, void *stream, const void *residual, void *ws, void *layer_out,
                    const FfnMlpWeights *w, int tokens, const FfnModelDims *dims);

/* Replaces forward_mlp_prepared (csrc/include/layers.h:330-333): as above from an already
 * normalized activation. */
int ffn_forward_mlp_prepared(void *cublas, void *stream, const void *normed, void *ws,
                             void *layer_out, const FfnMlpWeights *w, int tokens,
                             const FfnModelDims *dims);

/* Registers a k-major copy of a layer's down projection, which the decode kernels (1 or 2 tokens)
 * then use instead of the row-major matrix: WT [I/8][H] 32-bit words (word (kb, h) = the eight codes
 * k = 8kb..8kb+7 of output row h) and ST [I/128][H] scales, built on `stream` from the device buffers
 * w->down_i4 / w->down_i4_scales ([H][I/2], [H][I/128]; dims->intermediate_size is the rank-local I).
 * With it every CTA multiplies the down projection against only the act values it computed itself,
 * so the kernel needs no grid-wide hand-over between the two projections, and ffn_decode_stack runs
 * the whole stack in one persistent launch per 64 layers.  On B200 this kernel MEASURED SLOWER than
 * the row-major one (37.6 against 30.3 us on the 5120 x 17408 layer, 2628 against 2141 us for 64
 * layers), so preparing a layer is an opt-in for experiments, not a recommendation.  Results are not
 * bit-identical to the row-major kernel's (other summation order; same bars against the oracle).  The copy costs H*I/2 +
 * H*I/64 bytes of device memory per layer (+33 % of a layer's INT4 bytes) and is found again by the
 * ADDRESS w->down_i4: ffn_forward_mlp*, ffn_forward_mlp_tp, ffn_forward_mlp_host and ffn_decode_stack
 * use it whenever the layer they are given has one.  Call again after overwriting the weights, and
 * ffn_decode_layer_release before freeing them (a stale copy would be used for whatever is put at that
 * address next).  ffn_quantized_ffn_prepare_decode does it for every layer of a loaded handle (and the
 * handle's free releases them).  Layers without a copy
 * take the row-major kernel, which reads the reference's own uploads (csrc/engine.cu:2361-2401)
 * unchanged.  No counterpart in the reference. */
int ffn_decode_layer_prepare(const FfnMlpWeights *w, const FfnModelDims *dims, void *stream);
int ffn_decode_layer_release(const FfnMlpWeights *w);
int ffn_decode_layer_is_prepared(const FfnMlpWeights *w); /* 1 or 0 */
/* Launch geometry of the kernel over k-major copies, as ffn_int4_describe_plan gives it for the others. */
int ffn_int4_describe_kmajor_plan(int tokens, int hidden, int intermediate, int sm_count, int smem_optin, char *out,
                                  size_t out_bytes);

/* Which of the two kernels over k-major copies serves calls on prepared layers: 1 (default) the dp4a
 * kernel (16-bit block fixed point per 32 values, 1-2 tokens); 0 the variant whose inner products run
 * on the INT8 tensor cores (mma.sync m16n8k32, activations as two signed byte planes of 15-bit block
 * fixed point per 128 values, 1-4 tokens), falling back to the dp4a kernel for shapes it does not take.
 * The tensor-core variant measured slower on B200 (legacy mma.sync integer rate) and its coarser fixed
 * point leaves rare elements two BF16 steps from the reference's value over a 64-layer stack, so it is
 * opt-in and kept for A/B measurement.  Returns the previous setting. */
int ffn_int4_set_decode_kernel(int which);

/* Which pair of kernels serves 3..64 tokens per pass: 1 the mma.sync pair; 0 the tcgen05 pair
 * (tcgen05.mma with FP32 accumulators and the converted BF16 operand in tensor memory, packed INT4 rows
 * brought in by tiled TMA loads), falling back to the mma.sync pair for shapes it does not take (hidden
 * size not a multiple of 128, intermediate size not a multiple of 64); 2 (default) the tcgen05 pair
 * where it measured faster on B200 - more than 16 tokens and enough gate/up units (intermediate size / 64)
 * for half the SMs: 123 vs 186 us at 64 tokens, 93 vs 96 at 32 on the 5120 x 17408 layer, 114 vs 132 at
 * 64 tokens on its TP=2 slice - and the mma.sync pair elsewhere (73 vs 82 us at 16 tokens).  Same arithmetic in both: exact codes times BF16
 * activations summed in FP32 per 128-wide group, times the group's scale (the reference's tiled
 * kernel, csrc/kernels/gemm_quant.cu:134-147).  Returns the previous setting; any other value queries. */
int ffn_int4_set_batched_kernel(int which);

/* The layout the tcgen05 pair reads activations in ("tile order"), as arithmetic: byte offset of element
 * (token, k) of a bf16 [tokens][K] matrix whose token count is padded to `padded_tokens` (a multiple of
 * 16).  K runs in blocks of 64 values; inside a block a token owns a 128-byte row at
 * (token / 8) * 1024 + (token % 8) * 128, whose 16-byte piece c sits at piece c ^ (token % 8) (the
 * 128-byte swizzle of the MMA's shared-memory operand), the 8 values of a piece in the order
 * (0,4),(1,5),(2,6),(3,7).  -1 for arguments out of range.  Pure host arithmetic, no counterpart in
 * the reference. */
long long ffn_int4_tile_order_offset(int token, int k, int padded_tokens);

/* Overlap of consecutive FFN launches in one stream (default 1, on).  The fused FFN kernel is launched
 * with the programmatic-dependent-launch attribute: the next launch's CTAs are scheduled onto SMs as
 * this launch's CTAs leave them, set up their barriers and start the first copies of the weight stream,
 * and only then wait for this launch to complete before they touch the input, the workspace, the
 * output or the exchange slots.  The weight copies issued before that wait read the INT4 operands and
 * their scales, which therefore must not be written by the kernel that directly precedes the call in
 * the stream (the reference loads them once at start-up: csrc/safetensors_loader.cu); every other
 * operand may be.  0 turns the attribute off (plain cooperative launches, as CUDA orders them); any
 * other value queries.  Returns the previous setting.  The reference has no counterpart: its launches
 * are ordered by the stream alone (csrc/kernels/layers.cu:164, forward_mlp_prepared). */
int ffn_int4_set_launch_overlap(int on);

/* The fused FFN (as ffn_forward_mlp_prepared, 1 or 2 tokens) for callers that cannot allocate
 * device memory: a host that handed all of the GPU's memory to its own arena at start-up, so a
 * cudaMalloc from inside a library would fail, or a decode loop that cannot take the device-wide
 * synchronisation cudaMalloc and cudaFree imply.  This entry point calls no cudaMalloc, cudaFree or
 * other allocating routine and takes no workspace: the kernel's scratch (its synchronisation words
 * and the activation vector act that phase 1 passes to phase 2) sits in a fixed 128.25 KiB array
 * inside the library, which every GPU that loads the library holds until the process exits.
 * Limit: tokens * dims->intermediate_size <= 65536 (e.g. one token at I = 17408, two at I <= 32768);
 * larger requests are refused with FFN_ERR_CONFIG, as are shapes the fused kernel does not take.
 * The first call on each device looks up the array's device address (no allocation); make that
 * first call before any stream capture.  All calls on a device share the one array and it keeps the
 * last call's contents: the words that must start at zero are cleared on `stream` at the start of
 * every call, and two calls that overlap on the GPU (different streams) race - serialise them.
 * A bounded wait that ran out inside this entry point's kernel is reported by
 * ffn_int4_noalloc_status (which allocates nothing either); the status word is not cleared between
 * calls, so the report is not lost when further calls follow.
 * This entry point has no counterpart in the reference. */
int ffn_forward_mlp_prepared_noalloc(void *stream, const void *normed, void *layer_out,
                                     const FfnMlpWeights *w, int tokens, const FfnModelDims *dims);

/* ------------------------------------------------------------------------------------------- */
/* Tensor parallelism: the down projection's partial sums are reduced across ranks from inside    */
/* the FFN kernel (peer stores over NVLink), replacing allreduce_sum on the layer output           */
/* (csrc/include/layers.h:303-305; csrc/collective.cu:168-219; caller csrc/engine.cu:1436-1452)    */
/* and peer_probe_all (csrc/collective.cu:108-144).                                                */
/* ------------------------------------------------------------------------------------------- */
typedef struct FfnTpComm FfnTpComm;
#define FFN_TP_HANDLE_BYTES 64

/* Allocates this rank's exchange buffer on the current device (a call counter + 2*tp*max_tokens*hidden
 * 8-byte slots {FP32 partial sum, call number}, zeroed).  One communicator per rank; rank order is
 * device-list order as in the reference (csrc/engine.cu:997-1011). */
int ffn_tp_create(FfnTpComm **out, int tp, int rank, int hidden, int max_tokens);
/* One process per rank: export this rank's buffer (FFN_TP_HANDLE_BYTES bytes), exchange the handles
 * by any host channel, then connect with all tp handles in rank order (own entry ignored). */
int ffn_tp_export(FfnTpComm *comm, void *handle_out);
int ffn_tp_connect(FfnTpComm *comm, const void *all_handles);
/* One process driving every rank (the reference's process model, csrc/include/engine.h:8-9): enables
 * peer access between the communicators' devices and wires them up.  comms[i] must be rank i. */
int ffn_tp_connect_local(FfnTpComm *const *comms, int count);
int ffn_tp_destroy(FfnTpComm *comm);

/* One rank's FFN with the cross-rank reduce fused into the kernel: normed [tokens][H] (replicated on
 * every rank) -> layer_out [tokens][H] = bf16(sum over ranks of the FP32 down partials), identical on
 * every rank (partials are added in rank order).  `w`/`dims` describe the RANK-LOCAL operands
 * (gate/up [2*I/R][H], down [H][I/R], intermediate_size = I/R) exactly as the reference's per-rank
 * MlpWeights do.  `ws` as for ffn_forward_mlp.  If `residual` is non-NULL the kernel also applies
 * residual = bf16(f32(residual) + f32(layer_out)) (residual_add_device, csrc/engine.cu:1428-1433).
 * Every rank must make the same sequence of calls, each within about a second of the others; a rank
 * that never launches makes the others return after that bounded wait with a status
 * ffn_int4_device_status reports; after such a report the ranks' call counters may differ, so every
 * rank must either have made the same number of calls or destroy and recreate its communicator.  1 or 2 tokens run the single-launch kernel, 3..64 the tensor-core
 * pair (exchange in the down launch's epilogue); more are refused with FFN_ERR_CONFIG. */
int ffn_forward_mlp_tp(FfnTpComm *comm, void *stream, const void *normed, void *ws, void *layer_out,
                       const FfnMlpWeights *w, int tokens, const FfnModelDims *dims, void *residual);

/* The operator call for a caller whose activations live in HOST memory (the engine ABI's callers
 * pass host buffers, csrc/include/engine.h:11-12): copies normed_host [tokens][H] bf16 into
 * `staging`, runs ffn_forward_mlp_prepared (comm == NULL or one rank) or ffn_forward_mlp_tp on
 * `stream`, copies the result back to layer_out_host and synchronises the stream once - one call
 * instead of copy, launch, copy, synchronise issued separately.  `staging` is 2*tokens*H bf16 of
 * device memory owned by the caller; host buffers should be pinned (pageable memory works, through
 * the driver's staging).  Either host pointer may also be a device pointer.  No counterpart in the
 * reference (its decode step keeps activations on the device between sublayers). */
int ffn_forward_mlp_host(FfnTpComm *comm, void *stream, const void *normed_host, void *layer_out_host,
                         void *staging, void *ws, const FfnMlpWeights *w, int tokens, const FfnModelDims *dims);

/* Replaces allreduce_sum (csrc/include/layers.h:303-305; csrc/collective.cu:168-219) as a separate
 * collective, for the engine's other sharded sublayers and as the comparison arm of the fused
 * reduce: in-place elementwise sum of one buffer per rank over the communicator's exchange slots
 * (every rank pushes its elements into every rank's memory over NVLink, waits - bounded - for the
 * others', adds the tp values in rank order in FP32 and rounds once; the reference's leader adds
 * pairwise and rounds after every add).  dtype: 0 = float, 2 = bf16 (the values of COLLECTIVE_F32 /
 * COLLECTIVE_BF16, layers.h:272-278); other element types are refused with FFN_ERR_CONFIG as the
 * reference refuses unknown types.  `elements` may not exceed max_tokens * hidden of the communicator.
 * One rank per call; every rank makes the same call. */
int ffn_tp_allreduce_sum(FfnTpComm *comm, void *stream, void *buffer, size_t elements, int dtype);
/* The same for a process that drives every rank, in allreduce_sum's shape: comms[i], streams[i]
 * (may be NULL: default streams) and buffers[i] are index-aligned, comms[i] being rank i of `count`.
 * The reference's producer / done events and its leader staging buffer have no role here (ordering
 * is stream order, data goes straight into the peers' slots).  The caller synchronises afterwards. */
int ffn_allreduce_sum(FfnTpComm *const *comms, void *const *streams, int count, void *const *buffers,
                      size_t elements, int dtype);
/* The tag the exchange words of call number `call_number` carry (never zero, also across the wrap
 * of the 32-bit call counter).  Exported for tests; no counterpart in the reference. */
unsigned ffn_tp_exchange_tag(unsigned call_number);

/* The decode stack's FFN sublayers with identity mixers: for l in 0..num_layers-1,
 *     h <- bf16( f32(h) + f32( FFN_l( RMSNorm_l(h) ) ) )
 * which is what forward_replicated does per layer on this path - forward_ffn per rank, allreduce of
 * the layer output, residual_add_device (csrc/engine.cu:1603-1657, 1428-1452) - with the norm of
 * forward_mlp (csrc/kernels/layers.cu:149-160).  `layers[l]` are the rank-local operands including
 * post_norm_w; `h` is bf16 [tokens][H], updated in place and replicated on every rank; `layer_out`
 * receives the last layer's reduced FFN output; `ws` as for ffn_forward_mlp.  With 1 or 2 tokens a
 * layer is ONE kernel launch (norm, both projections, SiLU*up, cross-rank reduce and residual update
 * fused); with 3..64 tokens it is the norm kernel plus the tensor-core pair.  When every layer has a
 * k-major copy (ffn_decode_layer_prepare) and there are 1 or 2 tokens, the whole stack is ONE
 * persistent launch per 64 layers: the weight stream runs on through the layer boundaries while the
 * cross-rank exchange and the residual update of the previous layer are in flight.  comm == NULL or
 * a communicator of one rank means TP = 1.  Every rank makes the same call. */
int ffn_decode_stack(FfnTpComm *comm, void *stream, void *h, void *ws, void *layer_out,
                     const FfnMlpWeights *layers, int num_layers, int tokens, const FfnModelDims *dims);

/* ------------------------------------------------------------------------------------------- */
/* The artifact path: sidecar manifest, digests, shard views, per-rank load                        */
/* ------------------------------------------------------------------------------------------- */

/* Replaces sha256_hex (csrc/include/sha256.h; csrc/sha256.c): lower-case hex digest, NUL-terminated. */
int ffn_sha256_hex(const void *data, size_t len, char *out65);

/* Replaces quant_manifest_parse and its lookups (csrc/include/quant_manifest.h:121-137;
 * csrc/quant_manifest.c:895-1083).  These functions return the reference's QuantManifestStatus
 * values: 0 OK, 1 ARG, 2 SYNTAX, 3 FORMAT, 4 SHAPE, 5 IO, 6 HASH (quant_manifest.h:53-61); the
 * message is in ffn_int4_last_error().  Same schema and refusals: version 1, the frozen format block,
 * per entry packed.bytes == N*K/2, scales.count == N*K/128, scales.bytes == 2*count, dtypes u8/bf16,
 * 64 lower-case hex digests, a pair is its members' rows in order, the precision map and the entries
 * describe the same cells, duplicate keys / truncation / trailing bytes refused, at most 256 entries
 * and 128 pairs. */
typedef struct FfnQuantManifest FfnQuantManifest;
int ffn_quant_manifest_parse(const char *json, FfnQuantManifest **out);
void ffn_quant_manifest_free(FfnQuantManifest *manifest);
int ffn_quant_manifest_counts(const FfnQuantManifest *manifest, int *entries, int *pairs, int *int4_cells,
                              int *bf16_cells);
int ffn_quant_manifest_find_entry(const FfnQuantManifest *manifest, int layer, const char *role); /* index or -1 */
int ffn_quant_manifest_find_pair(const FfnQuantManifest *manifest, const char *name, int layer);  /* index or -1 */
int ffn_quant_manifest_entry_shape(const FfnQuantManifest *manifest, int index, long long *n, long long *k,
                                   long long *group, int *role_index);
int ffn_quant_manifest_pair_shape(const FfnQuantManifest *manifest, int index, long long *n, long long *k,
                                  long long *group);

/* Replaces quant_artifact_read (quant_manifest.h:139-143; csrc/quant_manifest.c:1085-1139): reads
 * root/file, requiring the expected dtype (want_dtype may be NULL: no expectation), then the recorded
 * size, then the SHA-256, in that order.
 * On success *out is a malloc'd buffer the caller releases with ffn_host_free; on refusal *out is NULL. */
int ffn_quant_artifact_read(const char *root, const char *file, const char *dtype, long long bytes,
                            const char *sha256, const char *want_dtype, uint8_t **out, size_t *out_len);
void ffn_host_free(void *p);

/* Replaces model_desc_shard_view for the two rules this path uses (csrc/model_desc.c:561-631):
 * rule 0 = none, 1 = OUT_DIM (rows split), 2 = IN_DIM (columns split).  view4 = {row_off, rows,
 * col_off, cols}.  Uneven splits and out-of-range ranks are refused (FFN_ERR_CONFIG). */
int ffn_shard_view(int rule, long long rows, long long cols, int tp, int rank, long long *view4);

/* Replaces the INT4 half of engine_load_quantized_ffn (csrc/include/engine.h:98;
 * csrc/engine.cu:2207-2428) for `num_layers` dense layers of shape hidden x intermediate (the whole,
 * unsliced intermediate size): reads manifest_dir/weights.manifest.json, requires an mlpGateUp pair
 * [2I, H] and an mlpDown entry [H, I] for every layer (all or nothing), verifies every artifact's size,
 * dtype and SHA-256 once, keeps rank `rank` of `tp`'s slice - gate rows and up rows
 * [rank*I/tp, (rank+1)*I/tp), down columns likewise, with the global scales those slices select;
 * a split that lands inside a 128-group is refused with "splits K at a non-group boundary" - and
 * uploads it to the current device through pinned staging.  FFN_ERR_WEIGHTS on any refusal. */
typedef struct FfnQuantizedFfn FfnQuantizedFfn;
int ffn_load_quantized_ffn(const char *manifest_dir, int num_layers, int hidden, int intermediate, int tp,
                           int rank, FfnQuantizedFfn **out);
/* The same for a process that drives every rank (the reference's model): reads and hashes each
 * artifact once and slices it for all `tp` ranks; out[r] lives on devices[r]. */
int ffn_load_quantized_ffn_ranks(const char *manifest_dir, int num_layers, int hidden, int intermediate,
                                 int tp, const int *devices, FfnQuantizedFfn **out);
/* Fills the INT4 members of `w` (gate_up_i4, its scales, down_i4, its scales, i4_group) with the
 * layer's device pointers, which stay owned by the handle (LayerWeights::owned, csrc/engine.cu:2184). */
int ffn_quantized_ffn_layer(const FfnQuantizedFfn *handle, int layer, FfnMlpWeights *w);
/* ffn_decode_layer_prepare for every layer of the handle, on the handle's device (opt-in; all or nothing).
 * No counterpart in the reference. */
int ffn_quantized_ffn_prepare_decode(FfnQuantizedFfn *handle);
int ffn_quantized_ffn_free(FfnQuantizedFfn *handle);

/* Replaces the reference's offline converter (scripts/quantize_weights.py:155-325, `convert`): reads the
 * BF16 safetensors shards of `model_dir` and the model descriptor (its num_layers, layer_ffns,
 * role_names and role_templates), quantizes the requested roles (NULL / 0 = mlpGate, mlpUp, mlpDown) of
 * every layer whose feed-forward is "dense" on the GPU with ffn_quantize_int4, and writes
 * `out_dir/weights.manifest.json` plus `out_dir/artifacts/<role>_layer<L>.{packed,scales}` and the
 * gate||up pair `mlpGateUp_layer<L>.*` (byte concatenation of its members), with the precision map,
 * the source files' sizes and digests (taken before and compared after), the descriptor's digest and
 * the quantization error against the source values.  The manifest is encoded as Python's
 * json.dump(indent=2, sort_keys=True) encodes it and is what ffn_quant_manifest_parse and the
 * reference's quant_manifest_parse accept; the artifacts are byte-identical to the reference
 * converter's.  limit_layers < 0 converts every layer, otherwise layers [0, limit_layers) as the
 * reference's --limit-layers does.  Refusals with the reference's wording: a non-BF16 source, a
 * tensor that is not 2-D, a tensor missing from the checkpoint or present in two shards, a
 * descriptor whose role names and templates differ, a source that changed during conversion, and
 * whatever the quantizer refuses. */
int ffn_convert_checkpoint(const char *model_dir, const char *descriptor_path, const char *out_dir,
                           const char *const *roles, int num_roles, int limit_layers);

/* Replaces the reference converter's --verify mode (scripts/quantize_weights.py:328-461): re-derives what
 * a manifest claims instead of trusting it.  Checks, in the reference's order and with its wording:
 * manifest version and the frozen format block; the source files still exist and hash as recorded;
 * no (layer, role) twice; shapes the format admits; every artifact present, of the recorded size and
 * digest; the descriptor's digest; the precision map covers every role of every layer exactly once
 * and agrees with the entries; every pair is its members' bytes in order and claims their combined
 * shape; and, when rederive_samples > 0, the first that many entries re-quantized from the source
 * checkpoint on the GPU are byte-identical to the artifacts (the reference samples two).  Returns the
 * number of problems found (0 = verified) or a negative status when the manifest cannot be read at
 * all; `report` receives one "verify: ..." line per problem, or the summary line. */
int ffn_verify_sidecar(const char *manifest_path, int rederive_samples, char *report, size_t report_bytes);

/* The converter's JSON encoder by itself: parses a document of numbers, strings, arrays and objects
 * and writes it back as json.dumps(indent=2, sort_keys=True) would (no trailing newline).  Exists so
 * the encoding can be compared with Python's without running a conversion; no counterpart in the
 * reference. */
int ffn_json_reencode(const char *json_in, char *out, size_t out_bytes);

/* ------------------------------------------------------------------------------------------- */
/* The reference's kernel test bridge (tests/kernels/kernel_bridge.cu), same names and           */
/* signatures, so the reference's own gate scripts can be pointed at this library.  Synchronous. */
/* Every pointer may be a host pointer or a device pointer; host buffers are staged.            */
/* ------------------------------------------------------------------------------------------- */
int test_gemm_int4(void *out, const void *a, const void *packed, const void *scales, int M, int N,
                   int K, int group);                                     /* kernel_bridge.cu:83-95 */
int test_silu_mul_packed(void *out, const void *packed, int tokens, int intermediate); /* :68-79 */
int test_norm(void *out, const void *x, const void *weight, int rows, int cols);       /* :31-41 */
int test_silu_mul(void *out, const void *gate, int n);                                  /* :55-66 */
int test_residual_norm(void *normed, void *residual, const void *sublayer, const void *weight, int hidden,
                       int rows, float eps, int gemma);                                 /* :99-113 */

#ifdef __cplusplus
}
#endif

#endif /* FFN_INT4_H */
