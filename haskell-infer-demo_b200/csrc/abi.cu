/*
 * abi.cu - the extern "C" surface of libffn_int4.so (declared in include/ffn_int4.h): argument
 * validation in the reference's order, status codes instead of exceptions, and the reference's
 * kernel test bridge names.
 */
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <new>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace ffn {

#define FFN_INT4_STR2(x) #x
#define FFN_INT4_STR(x) FFN_INT4_STR2(x)
static thread_local char g_error[512];
static int g_fused_enabled = 1;

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

void clear_error() { g_error[0] = '\0'; }

/* Validation shared by the GEMM entry points; mirrors gemm_int4_bf16's checks
 * (csrc/kernels/gemm_quant.cu:208-224).  Returns 1 for "nothing to do". */
static int check_gemm(const char *who, const void *a, const void *packed, const void *scales,
                      const void *out, int M, int N, int K, int group) {
    if (M < 0 || N < 0 || K <= 0 || group <= 0)
        return fail(FFN_ERR_CONFIG, "%s: negative extent or nonpositive group", who);
    if (M == 0 || N == 0) return 1;
    if (!a || !packed || !scales || !out) return fail(FFN_ERR_CONFIG, "%s: null buffer", who);
    if (K % group != 0)
        return fail(FFN_ERR_CONFIG, "%s: K=%d is not a whole number of %d-wide groups", who, K, group);
    if (group != FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "%s: this format's group is %d, not %d", who, FFN_INT4_GROUP, group);
    if (((uintptr_t)packed & 15) || ((uintptr_t)a & 15))
        return fail(FFN_ERR_CONFIG, "%s: the activation and the packed weight must be 16-byte aligned", who);
    return FFN_OK;
}

static int mlp_common(cudaStream_t stream, const void *normed, void *ws, void *layer_out,
                      const FfnMlpWeights *w, int tokens, const FfnModelDims *dims) {
    const int H = dims->hidden_size, I = dims->intermediate_size;
    uint16_t *base = (uint16_t *)ws;
    uint16_t *packed_act = base + (size_t)tokens * H;            /* [T, 2I] gate|up */
    uint16_t *act = packed_act + (size_t)2 * tokens * I;         /* [T, I] */
    int st = g_fused_enabled ? fused_ffn_try(stream, normed, act, layer_out, w, tokens, H, I) : FFN_NOT_ADMITTED;
    if (st != FFN_NOT_ADMITTED) return st;
    if (g_fused_enabled) { /* 3..64 tokens per pass on the tensor cores; longer batches in blocks of 64 */
        unsigned *status = nullptr;
        if ((st = fused_status_word(&status))) return st;
        bool taken = true;
        for (int m0 = 0; m0 < tokens && taken; m0 += 64) {
            const int m = tokens - m0 < 64 ? tokens - m0 : 64;
            st = batched_ffn_launch(stream, (const uint16_t *)normed + (size_t)m0 * H, act + (size_t)m0 * I,
                                (uint16_t *)layer_out + (size_t)m0 * H, w, m, H, I, nullptr, nullptr, status);
            if (st == FFN_NOT_ADMITTED) { taken = false; break; }
            if (st) return st;
        }
        if (taken) return FFN_OK;
        if (tokens > 64) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp: the batched kernel does not take this shape");
    }
    st = gemm_int4_generic(normed, w->gate_up_i4, w->gate_up_i4_scales, packed_act, nullptr, tokens,
                           2 * I, H, stream);
    if (st) return st;
    st = silu_mul_packed(act, packed_act, tokens, I, stream);
    if (st) return st;
    return gemm_int4_generic(act, w->down_i4, w->down_i4_scales, layer_out, nullptr, tokens, H, I,
                             stream);
}

static int check_mlp(const char *who, const void *in, const void *ws, const void *layer_out,
                     const FfnMlpWeights *w, int tokens, const FfnModelDims *dims) {
    if (!dims || !w) return fail(FFN_ERR_CONFIG, "%s: null weights or dims", who);
    const int limit = dims->max_chunk > 0 ? dims->max_chunk : 128; /* ENGINE_MAX_CHUNK, layers.h:51 */
    if (tokens < 1 || tokens > limit)
        return fail(FFN_ERR_CONFIG, "%s: Layer token count exceeds the model's max_chunk", who);
    if (!in || !ws || !layer_out) return fail(FFN_ERR_CONFIG, "%s: null buffer", who);
    if (!w->gate_up_i4 || !w->gate_up_i4_scales || !w->down_i4 || !w->down_i4_scales)
        return fail(FFN_ERR_CONFIG, "%s: the layer carries no INT4 operands (this library has no BF16 path)", who);
    if (w->i4_group != FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "%s: this format's group is %d, not %d", who, FFN_INT4_GROUP, w->i4_group);
    const int H = dims->hidden_size, I = dims->intermediate_size;
    if (H <= 0 || I <= 0 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "%s: hidden=%d / intermediate=%d are not whole numbers of %d-wide groups",
                    who, H, I, FFN_INT4_GROUP);
    return FFN_OK;
}

/* A host-or-device pointer made device-resident for the synchronous test bridge. */
struct Staged {
    void *dev = nullptr;
    void *host = nullptr;
    size_t bytes = 0;
    bool owned = false;
    bool writeback = false;
    int acquire(const void *p, size_t n, bool is_output) {
        bytes = n;
        cudaPointerAttributes attr;
        cudaError_t e = cudaPointerGetAttributes(&attr, p);
        if (e != cudaSuccess) { (void)cudaGetLastError(); attr.type = cudaMemoryTypeUnregistered; }
        if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
            dev = const_cast<void *>(p);
            return FFN_OK;
        }
        host = const_cast<void *>(p);
        owned = true;
        writeback = is_output;
        if (cudaMalloc(&dev, n ? n : 1) != cudaSuccess) return fail(FFN_ERR_ALLOC, "test bridge: cudaMalloc(%zu) failed", n);
        if (!is_output) FFN_CUDA_TRY(cudaMemcpy(dev, p, n, cudaMemcpyHostToDevice), "test bridge: upload");
        return FFN_OK;
    }
    int finish() {
        if (owned && writeback) FFN_CUDA_TRY(cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost), "test bridge: download");
        return FFN_OK;
    }
    ~Staged() { if (owned && dev) cudaFree(dev); }
};

}  // namespace ffn

using namespace ffn;

extern "C" {

const char *ffn_int4_last_error(void) { return g_error; }
int ffn_int4_abi_version(void) { return FFN_INT4_ABI_VERSION; }

int ffn_int4_describe_plan(int tokens, int hidden, int intermediate, int sm_count, int smem_optin, char *out,
                           size_t out_bytes) {
    clear_error();
    if (!out || out_bytes < 64) return fail(FFN_ERR_CONFIG, "ffn_int4_describe_plan: the text buffer is too small");
    if (tokens < 1 || hidden <= 0 || intermediate <= 0 || hidden % FFN_INT4_GROUP || intermediate % FFN_INT4_GROUP ||
        sm_count < 1 || smem_optin < 1)
        return fail(FFN_ERR_CONFIG, "ffn_int4_describe_plan: invalid shape or device description");
    if (tokens <= 2 && fused_describe_plan(tokens, hidden, intermediate, sm_count, smem_optin, out, out_bytes)) return FFN_OK;
    if (tc_describe_plan(tokens < 64 ? tokens : 64, hidden, intermediate, sm_count, smem_optin, out, out_bytes) ||
        mma_describe_plan(tokens < 64 ? tokens : 64, hidden, intermediate, sm_count, smem_optin, out, out_bytes)) {
        if (tokens > 64) { /* longer batches go through the pair in blocks of 64 tokens */
            const size_t used = strlen(out);
            snprintf(out + used, out_bytes - used, " passes=%d", (tokens + 63) / 64);
        }
        return FFN_OK;
    }
    snprintf(out, out_bytes, "kernel=generic launches=3 (gate/up GEMM, SiLU*up, down GEMM)");
    return FFN_OK;
}

int ffn_int4_describe_kmajor_plan(int tokens, int hidden, int intermediate, int sm_count, int smem_optin, char *out,
                                  size_t out_bytes) {
    clear_error();
    if (!out || out_bytes < 64) return fail(FFN_ERR_CONFIG, "ffn_int4_describe_kmajor_plan: the text buffer is too small");
    if (tokens < 1 || hidden <= 0 || intermediate <= 0 || hidden % FFN_INT4_GROUP || intermediate % FFN_INT4_GROUP ||
        sm_count < 1 || smem_optin < 1)
        return fail(FFN_ERR_CONFIG, "ffn_int4_describe_kmajor_plan: invalid shape or device description");
    if (imma_describe_plan(tokens, hidden, intermediate, sm_count, smem_optin, out, out_bytes)) return FFN_OK;
    if (kmajor_describe_plan(tokens, hidden, intermediate, sm_count, smem_optin, out, out_bytes)) return FFN_OK;
    snprintf(out, out_bytes, "kernel=none (the k-major kernel does not take this shape; the row-major kernels do)");
    return FFN_OK;
}

int ffn_int4_set_decode_kernel(int which) {
    if (which != 0 && which != 1) { /* a query: leaves the setting as it is */
        const int current = kmajor_prefer_dp4a(1);
        kmajor_prefer_dp4a(current);
        return current;
    }
    return kmajor_prefer_dp4a(which);
}

int ffn_int4_set_batched_kernel(int which) {
    if (which < 0 || which > 2) { /* a query */
        const int mode = tc_set_mode(2);
        tc_set_mode(mode);
        return mode;
    }
    return tc_set_mode(which);
}

long long ffn_int4_tile_order_offset(int token, int k, int padded_tokens) {
    if (token < 0 || k < 0 || padded_tokens < 16 || padded_tokens % 16 || token >= padded_tokens) return -1;
    return tc_tile_order_offset(token, k, padded_tokens);
}

int ffn_int4_set_launch_overlap(int on) {
    if (on != 0 && on != 1) {
        const int current = fused_set_launch_overlap(1);
        fused_set_launch_overlap(current);
        return current;
    }
    return fused_set_launch_overlap(on);
}

int ffn_int4_describe_gemm_plan(int m, int n, int k, int sm_count, int smem_optin, char *out, size_t out_bytes) {
    clear_error();
    if (!out || out_bytes < 64) return fail(FFN_ERR_CONFIG, "ffn_int4_describe_gemm_plan: the text buffer is too small");
    if (m < 1 || n <= 0 || k <= 0 || k % FFN_INT4_GROUP || sm_count < 1 || smem_optin < 1)
        return fail(FFN_ERR_CONFIG, "ffn_int4_describe_gemm_plan: invalid shape or device description");
    if (m <= 2 && gemv_describe_plan(m, n, k, sm_count, smem_optin, out, out_bytes)) return FFN_OK;
    snprintf(out, out_bytes, "kernel=generic launches=1");
    return FFN_OK;
}

int ffn_int4_set_fused(int enabled) {
    const int old = g_fused_enabled;
    g_fused_enabled = enabled != 0;
    return old;
}

void ffn_int4_debug_trace(void *device_buffer) { fused_set_trace((long long *)device_buffer); }

static int report_status(unsigned st, int *where, int *cta) {
    if (where) *where = (int)(st & 0xFF);
    if (cta) *cta = (int)(st >> 8);
    if (st != 0) {
        static const char *names[] = {"", "producer waiting for a free stage", "consumer waiting for weights",
                                      "consumer waiting for a partial slot", "epilogue waiting for partials",
                                      "grid barrier", "a peer rank's partial sums", "draining copies",
                                      "consumer waiting for the activation vector", "waiting for the other CTAs' partial sums",
                                      "waiting for the residual stream of the next layer", "waiting for this CTA's own activations",
                                      "", "", "", "", "", "", "", "",
                                      "tcgen05 producer waiting for a free stage", "tcgen05 kernel waiting for a stage's copies",
                                      "conversion warps waiting for a free operand buffer", "MMA thread waiting for a converted operand",
                                      "MMA thread waiting for a free accumulator", "epilogue waiting for an accumulator"};
        const unsigned w = st & 0xFF;
        return fail(FFN_ERR_CUDA, "a bounded device-side wait ran out (%s, CTA %u); the kernel returned early and "
                    "its output is invalid", w < sizeof(names) / sizeof(names[0]) ? names[w] : "unknown", st >> 8);
    }
    return FFN_OK;
}

int ffn_int4_device_status(int *where, int *cta) {
    clear_error();
    unsigned st = 0;
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(FFN_ERR_CUDA, "ffn_int4_device_status: %s", cudaGetErrorString(e));
    int rc = fused_status(&st, true);
    if (rc) return rc;
    if (st == 0 && fused_noalloc_in_use()) { /* the allocation-free entry point keeps its own status word */
        rc = fused_status_noalloc(&st, true);
        if (rc) return rc;
    }
    return report_status(st, where, cta);
}

int ffn_int4_noalloc_status(int *where, int *cta) {
    clear_error();
    unsigned st = 0;
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(FFN_ERR_CUDA, "ffn_int4_noalloc_status: %s", cudaGetErrorString(e));
    const int rc = fused_status_noalloc(&st, true);
    if (rc) return rc;
    return report_status(st, where, cta);
}

unsigned ffn_tp_exchange_tag(unsigned call_number) { return tp_tag(call_number); }

const char *ffn_int4_numerical_policy(void) {
    /* Sorted keys, no whitespace: ready to be spliced into the fields of a numerical_policy block. */
    return "\"ffn_int4_accumulate\":\"block_fixed_point_a16_dp4a_per_32_fp32_across;mma_bf16_codes_fp32_per_group\","
           "\"ffn_int4_kernel\":\"b200_ffn_int4_abi" FFN_INT4_STR(FFN_INT4_ABI_VERSION) "\","
           "\"ffn_int4_roundings\":\"gate_up_bf16;silu_mul_bf16;down_bf16_after_reduce\","
           "\"ffn_tp_reduce\":\"fp32_partials_rank_order_single_rounding\","
           "\"weight_quantization\":\"int4_symmetric_group_bf16_scale_decode_only\"";
}

int ffn_gemm_int4_bf16(const void *a, const void *packed, const void *scales, void *out, int M, int N,
                       int K, int group, void *stream) {
    clear_error();
    const int c = check_gemm("ffn_gemm_int4_bf16", a, packed, scales, out, M, N, K, group);
    if (c == 1) return FFN_OK;
    if (c) return c;
    return gemm_int4_dispatch(a, packed, scales, out, M, N, K, (cudaStream_t)stream);
}

int ffn_silu_mul_packed(void *out, const void *packed, int tokens, int intermediate, void *stream) {
    clear_error();
    if (tokens < 0 || intermediate < 0) return fail(FFN_ERR_CONFIG, "ffn_silu_mul_packed: negative extent");
    if (tokens == 0 || intermediate == 0) return FFN_OK;
    if (!out || !packed) return fail(FFN_ERR_CONFIG, "ffn_silu_mul_packed: null buffer");
    return silu_mul_packed(out, packed, tokens, intermediate, (cudaStream_t)stream);
}

int ffn_gemma_rms_norm(void *out, const void *x, const void *weight, int cols, int rows, float eps,
                       void *stream) {
    clear_error();
    if (rows < 0 || cols <= 0 || !(eps > 0.0f) || !(eps < 3.0e38f))
        return fail(FFN_ERR_CONFIG, "ffn_gemma_rms_norm: invalid shape or epsilon");
    if (rows == 0) return FFN_OK;
    if (!out || !x || !weight) return fail(FFN_ERR_CONFIG, "ffn_gemma_rms_norm: null buffer");
    return gemma_rms_norm(out, x, weight, cols, rows, eps, 1, (cudaStream_t)stream);
}

int ffn_residual_norm(void *normed, void *residual, const void *sublayer, const void *weight, int hidden, int rows,
                      float eps, int gemma, void *stream) {
    clear_error();
    if (hidden <= 0 || rows < 0 || !(eps > 0.0f) || !(eps < 3.0e38f))
        return fail(FFN_ERR_CONFIG, "ffn_residual_norm: invalid shape or epsilon");
    if (rows == 0) return FFN_OK;
    if (!normed || !residual || !sublayer || !weight) return fail(FFN_ERR_CONFIG, "ffn_residual_norm: null buffer");
    return residual_norm(normed, residual, sublayer, weight, hidden, rows, eps, gemma ? 1 : 0, (cudaStream_t)stream);
}

int ffn_silu_mul(void *out, const void *gate, int n, void *stream) {
    clear_error();
    if (n < 0) return fail(FFN_ERR_CONFIG, "ffn_silu_mul: negative element count");
    if (n == 0) return FFN_OK;
    if (!out || !gate) return fail(FFN_ERR_CONFIG, "ffn_silu_mul: expected contiguous [gate[n], up[n]] input");
    if (n >= 8 && (n % 8 != 0 || ((uintptr_t)gate & 15) || ((uintptr_t)out & 15)))
        return fail(FFN_ERR_CONFIG, "ffn_silu_mul: vectorized input/output must be 16-byte aligned and n divisible by 8");
    return silu_mul_pair(out, gate, n, (cudaStream_t)stream);
}

int ffn_residual_add(void *dst, const void *src, int n, void *stream) {
    clear_error();
    if (n < 0) return fail(FFN_ERR_CONFIG, "ffn_residual_add: negative element count");
    if (n == 0) return FFN_OK;
    if (!dst || !src) return fail(FFN_ERR_CONFIG, "ffn_residual_add: null buffer");
    return residual_add(dst, src, n, (cudaStream_t)stream);
}

int ffn_dequantize_int4(void *out, const void *packed, const void *scales, int N, int K, int *bad,
                        void *stream) {
    clear_error();
    if (N <= 0 || K <= 0 || K % FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "ffn_dequantize_int4: the format cannot hold [%d, %d]", N, K);
    if (!out || !packed || !scales) return fail(FFN_ERR_CONFIG, "ffn_dequantize_int4: null buffer");
    return dequantize_int4(out, packed, scales, N, K, bad, (cudaStream_t)stream);
}

int ffn_forward_mlp(void *cublas, void *stream, const void *residual, void *ws, void *layer_out,
                    const FfnMlpWeights *w, int tokens, const FfnModelDims *dims) {
    (void)cublas;
    clear_error();
    const int c = check_mlp("ffn_forward_mlp", residual, ws, layer_out, w, tokens, dims);
    if (c) return c;
    const void *normed = residual;
    if (w->post_norm_w) {
        if (!(dims->rms_eps > 0.0f)) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp: invalid shape or epsilon");
        const int st = gemma_rms_norm(ws, residual, w->post_norm_w, dims->hidden_size, tokens,
                                      dims->rms_eps, dims->norm_style == 0, (cudaStream_t)stream);
        if (st) return st;
        normed = ws;
    }
    return mlp_common((cudaStream_t)stream, normed, ws, layer_out, w, tokens, dims);
}

int ffn_forward_mlp_prepared(void *cublas, void *stream, const void *normed, void *ws, void *layer_out,
                             const FfnMlpWeights *w, int tokens, const FfnModelDims *dims) {
    (void)cublas;
    clear_error();
    const int c = check_mlp("ffn_forward_mlp_prepared", normed, ws, layer_out, w, tokens, dims);
    if (c) return c;
    return mlp_common((cudaStream_t)stream, normed, ws, layer_out, w, tokens, dims);
}

int ffn_forward_mlp_prepared_noalloc(void *stream, const void *normed, void *layer_out,
                                     const FfnMlpWeights *w, int tokens, const FfnModelDims *dims) {
    clear_error();
    if (!dims || !w) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: null weights or dims");
    if (!normed || !layer_out) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: null buffer");
    if (!w->gate_up_i4 || !w->gate_up_i4_scales || !w->down_i4 || !w->down_i4_scales)
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: the layer carries no INT4 operands");
    if (w->i4_group != FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: this format's group is %d, not %d", FFN_INT4_GROUP, w->i4_group);
    const int H = dims->hidden_size, I = dims->intermediate_size;
    if (H <= 0 || I <= 0 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_prepared_noalloc: hidden=%d / intermediate=%d are not whole numbers "
                    "of %d-wide groups", H, I, FFN_INT4_GROUP);
    return fused_ffn_launch_noalloc((cudaStream_t)stream, normed, layer_out, w, tokens, H, I);
}

/* ---- the reference's kernel test bridge ---------------------------------------------------- */

int test_gemm_int4(void *out, const void *a, const void *packed, const void *scales, int M, int N,
                   int K, int group) {
    clear_error();
    const int c = check_gemm("test_gemm_int4", a ? a : (const void *)16, packed ? packed : (const void *)16,
                             scales, out, M, N, K, group);
    if (c == 1) return 0;
    if (c) { fprintf(stderr, "test_gemm_int4: %s\n", g_error); return -1; }
    if (!a || !packed) { fprintf(stderr, "test_gemm_int4: null buffer\n"); return -1; }
    Staged so, sa, sp, ss;
    int st = so.acquire(out, (size_t)M * N * 2, true);
    if (!st) st = sa.acquire(a, (size_t)M * K * 2, false);
    if (!st) st = sp.acquire(packed, (size_t)N * K / 2, false);
    if (!st) st = ss.acquire(scales, (size_t)N * (K / group) * 2, false);
    if (!st) st = gemm_int4_dispatch(sa.dev, sp.dev, ss.dev, so.dev, M, N, K, nullptr);
    if (st) { fprintf(stderr, "test_gemm_int4: %s\n", g_error); return -1; }
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    return so.finish() ? -1 : 0;
}

int test_silu_mul_packed(void *out, const void *packed, int tokens, int intermediate) {
    clear_error();
    if (tokens < 0 || intermediate < 0) { fprintf(stderr, "test_silu_mul_packed: negative extent\n"); return -1; }
    if (tokens == 0 || intermediate == 0) return 0;
    if (!out || !packed) { fprintf(stderr, "test_silu_mul_packed: null buffer\n"); return -1; }
    Staged so, sp;
    int st = so.acquire(out, (size_t)tokens * intermediate * 2, true);
    if (!st) st = sp.acquire(packed, (size_t)tokens * intermediate * 4, false);
    if (!st) st = silu_mul_packed(so.dev, sp.dev, tokens, intermediate, nullptr);
    if (st) { fprintf(stderr, "test_silu_mul_packed: %s\n", g_error); return -1; }
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    return so.finish() ? -1 : 0;
}

int test_silu_mul(void *out, const void *gate, int n) {
    clear_error();
    if (n < 0) { fprintf(stderr, "test_silu_mul: negative element count\n"); return -1; }
    if (n == 0) return 0;
    Staged so, sg;
    int st = so.acquire(out, (size_t)n * 2, true);
    if (!st) st = sg.acquire(gate, (size_t)n * 4, false);
    if (!st) st = ffn_silu_mul(so.dev, sg.dev, n, nullptr);
    if (st) { fprintf(stderr, "test_silu_mul: %s\n", g_error); return -1; }
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    return so.finish() ? -1 : 0;
}

int test_residual_norm(void *normed, void *residual, const void *sublayer, const void *weight, int hidden, int rows,
                       float eps, int gemma) {
    clear_error();
    if (hidden <= 0 || rows < 0) { fprintf(stderr, "test_residual_norm: invalid shape or epsilon\n"); return -1; }
    if (rows == 0) return 0;
    if (!normed || !residual || !sublayer || !weight) { fprintf(stderr, "test_residual_norm: null buffer\n"); return -1; }
    const size_t bytes = (size_t)rows * hidden * 2;
    Staged sn, sr, ss, sw;
    int st = sn.acquire(normed, bytes, true);
    if (!st) st = sr.acquire(residual, bytes, false);
    if (!st) st = ss.acquire(sublayer, bytes, false);
    if (!st) st = sw.acquire(weight, (size_t)hidden * 2, false);
    sr.writeback = sr.owned; /* the residual is both input and output */
    if (!st) st = ffn_residual_norm(sn.dev, sr.dev, ss.dev, sw.dev, hidden, rows, eps, gemma, nullptr);
    if (st) { fprintf(stderr, "test_residual_norm: %s\n", g_error); return -1; }
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    return (sn.finish() || sr.finish()) ? -1 : 0;
}

int test_norm(void *out, const void *x, const void *weight, int rows, int cols) {
    clear_error();
    if (rows < 0 || cols <= 0) { fprintf(stderr, "test_norm: invalid shape or epsilon\n"); return -1; }
    if (rows == 0) return 0;
    if (!out || !x || !weight) { fprintf(stderr, "test_norm: null buffer\n"); return -1; }
    Staged so, sx, sw;
    int st = so.acquire(out, (size_t)rows * cols * 2, true);
    if (!st) st = sx.acquire(x, (size_t)rows * cols * 2, false);
    if (!st) st = sw.acquire(weight, (size_t)cols * 2, false);
    if (!st) st = gemma_rms_norm(so.dev, sx.dev, sw.dev, cols, rows, 1e-6f, 1, nullptr);
    if (st) { fprintf(stderr, "test_norm: %s\n", g_error); return -1; }
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    return so.finish() ? -1 : 0;
}

}  // extern "C"
