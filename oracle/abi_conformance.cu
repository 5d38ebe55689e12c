/*
 * abi_conformance.cu - TEST INFRASTRUCTURE ONLY: compiled (never linked, never run) where a checkout
 * of the reference is present, so that drift between include/ffn_int4.h and the reference's own
 * headers breaks the build instead of corrupting a struct at run time.  The precedent is the
 * reference's engine stub, which includes engine.h for the same reason
 * (tests/generation_engine_stub.c:1-12).
 *
 * Checked: every field of FfnMlpWeights / FfnModelDims sits at the offset and has the size of the
 * same-named field of MlpWeights / ModelDims (csrc/include/layers.h:18-47, 54-70), so the engine can
 * pass its own structs; the status codes equal ENGINE_OK / ENGINE_ERR_* (csrc/include/engine.h:264-270);
 * the collective dtype values ffn_tp_allreduce_sum takes equal COLLECTIVE_F32 / COLLECTIVE_BF16
 * (layers.h:272-278); the format constants equal the frozen ones (csrc/include/linear_weight.h:46-54);
 * and the reference's operator prototypes still have the argument lists the replacements mirror.
 */
#include <cstddef>
#include <type_traits>

#include "layers.h"        /* the reference's: -I<reference>/csrc/include */
#include "engine.h"
#include "linear_weight.h"
#include "quant_manifest.h"

#include "../include/ffn_int4.h"

#define SAME_FIELD(Ours, Theirs, f)                                                        \
    static_assert(offsetof(Ours, f) == offsetof(Theirs, f), #Ours "." #f ": offset drifted"); \
    static_assert(sizeof(((Ours *)0)->f) == sizeof(((Theirs *)0)->f), #Ours "." #f ": size drifted")

static_assert(sizeof(FfnMlpWeights) == sizeof(MlpWeights), "MlpWeights mirror: size drifted");
SAME_FIELD(FfnMlpWeights, MlpWeights, gate_proj_w);
SAME_FIELD(FfnMlpWeights, MlpWeights, up_proj_w);
SAME_FIELD(FfnMlpWeights, MlpWeights, down_proj_w);
SAME_FIELD(FfnMlpWeights, MlpWeights, post_norm_w);
SAME_FIELD(FfnMlpWeights, MlpWeights, gate_up_i4);
SAME_FIELD(FfnMlpWeights, MlpWeights, gate_up_i4_scales);
SAME_FIELD(FfnMlpWeights, MlpWeights, down_i4);
SAME_FIELD(FfnMlpWeights, MlpWeights, down_i4_scales);
SAME_FIELD(FfnMlpWeights, MlpWeights, i4_group);

static_assert(sizeof(FfnModelDims) == sizeof(ModelDims), "ModelDims mirror: size drifted");
SAME_FIELD(FfnModelDims, ModelDims, hidden_size);
SAME_FIELD(FfnModelDims, ModelDims, intermediate_size);
SAME_FIELD(FfnModelDims, ModelDims, num_heads);
SAME_FIELD(FfnModelDims, ModelDims, num_kv_heads);
SAME_FIELD(FfnModelDims, ModelDims, head_dim);
SAME_FIELD(FfnModelDims, ModelDims, rotary_dim);
SAME_FIELD(FfnModelDims, ModelDims, norm_style);
SAME_FIELD(FfnModelDims, ModelDims, attn_output_gate);
SAME_FIELD(FfnModelDims, ModelDims, q_gate_interleave);
SAME_FIELD(FfnModelDims, ModelDims, num_layers);
SAME_FIELD(FfnModelDims, ModelDims, vocab_size);
SAME_FIELD(FfnModelDims, ModelDims, rms_eps);
SAME_FIELD(FfnModelDims, ModelDims, rope_theta);
SAME_FIELD(FfnModelDims, ModelDims, max_seq_len);
SAME_FIELD(FfnModelDims, ModelDims, gdn_conv_dim);
SAME_FIELD(FfnModelDims, ModelDims, gdn_value_dim);
SAME_FIELD(FfnModelDims, ModelDims, gdn_num_v_heads);
SAME_FIELD(FfnModelDims, ModelDims, gdn_num_k_heads);
SAME_FIELD(FfnModelDims, ModelDims, gdn_head_dim);
SAME_FIELD(FfnModelDims, ModelDims, gdn_conv_kernel);
SAME_FIELD(FfnModelDims, ModelDims, mla_kv_lora_rank);
SAME_FIELD(FfnModelDims, ModelDims, mla_qk_nope_head_dim);
SAME_FIELD(FfnModelDims, ModelDims, mla_qk_rope_head_dim);
SAME_FIELD(FfnModelDims, ModelDims, mla_v_head_dim);
SAME_FIELD(FfnModelDims, ModelDims, max_chunk);
static_assert(std::is_same<decltype(ModelDims::rms_eps), float>::value, "rms_eps is read as a float");

static_assert(FFN_OK == ENGINE_OK && FFN_ERR_CUDA == ENGINE_ERR_CUDA && FFN_ERR_ALLOC == ENGINE_ERR_ALLOC &&
              FFN_ERR_WEIGHTS == ENGINE_ERR_WEIGHTS && FFN_ERR_CONFIG == ENGINE_ERR_CONFIG &&
              FFN_ERR_STATE == ENGINE_ERR_STATE, "status codes drifted from engine.h");
static_assert(COLLECTIVE_F32 == 0 && COLLECTIVE_BF16 == 2, "collective element tags drifted");
static_assert(FFN_INT4_GROUP == LINEAR_WEIGHT_GROUP_SIZE, "format group drifted");
static_assert(ENGINE_MAX_CHUNK == 128, "default max_chunk drifted");

/* The reference's operator prototypes, as the replacements mirror them (argument order and types).
 * Assigning the functions to pointers of the expected types fails to compile when a prototype moves. */
static int (*const check_forward_mlp)(cublasHandle_t, cudaStream_t, const __nv_bfloat16 *, __nv_bfloat16 *, __nv_bfloat16 *,
                                      const MlpWeights *, int, const ModelDims *) = &forward_mlp;
static int (*const check_forward_mlp_prepared)(cublasHandle_t, cudaStream_t, const __nv_bfloat16 *, __nv_bfloat16 *,
                                               __nv_bfloat16 *, const MlpWeights *, int, const ModelDims *) = &forward_mlp_prepared;
static int (*const check_gemm_int4)(const __nv_bfloat16 *, const uint8_t *, const __nv_bfloat16 *, __nv_bfloat16 *, int, int,
                                    int, int, cudaStream_t) = &gemm_int4_bf16;
static int (*const check_allreduce)(const int *, cudaStream_t *, cudaEvent_t *, cudaEvent_t *, int, void *const *, void *,
                                    size_t, CollectiveDtype) = &allreduce_sum;
static int (*const check_load)(EngineHandle *, const char *) = &engine_load_quantized_ffn;

/* Our replacements, with the same argument order (pointers as void *, status instead of exceptions). */
static int (*const ours_forward_mlp)(void *, void *, const void *, void *, void *, const FfnMlpWeights *, int,
                                     const FfnModelDims *) = &ffn_forward_mlp;
static int (*const ours_gemm)(const void *, const void *, const void *, void *, int, int, int, int, void *) = &ffn_gemm_int4_bf16;

int ffn_int4_abi_conformance_anchor(void) {
    return (check_forward_mlp && check_forward_mlp_prepared && check_gemm_int4 && check_allreduce && check_load &&
            ours_forward_mlp && ours_gemm) ? 0 : 1;
}
