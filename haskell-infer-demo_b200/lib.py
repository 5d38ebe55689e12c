"""ctypes binding of libffn_int4.so.  Fails loudly when the library is absent."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libffn_int4.so")
HEADER = os.path.join(HERE, "..", "include", "ffn_int4.h")
_lib = None


class LibraryMissing(RuntimeError):
    pass


class FfnError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"libffn_int4 status {status}: {message}")
        self.status = status
        self.message = message


class MlpWeights(ctypes.Structure):
    """Mirror of FfnMlpWeights (= the reference's MlpWeights, csrc/include/layers.h:54-70)."""
    _fields_ = [("gate_proj_w", ctypes.c_void_p), ("up_proj_w", ctypes.c_void_p),
                ("down_proj_w", ctypes.c_void_p), ("post_norm_w", ctypes.c_void_p),
                ("gate_up_i4", ctypes.c_void_p), ("gate_up_i4_scales", ctypes.c_void_p),
                ("down_i4", ctypes.c_void_p), ("down_i4_scales", ctypes.c_void_p),
                ("i4_group", ctypes.c_int)]


class ModelDims(ctypes.Structure):
    """Mirror of FfnModelDims (= the reference's ModelDims, csrc/include/layers.h:19-47)."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "hidden_size", "intermediate_size", "num_heads", "num_kv_heads", "head_dim", "rotary_dim",
        "norm_style", "attn_output_gate", "q_gate_interleave", "num_layers", "vocab_size")] + \
        [("rms_eps", ctypes.c_float), ("rope_theta", ctypes.c_float)] + \
        [(n, ctypes.c_int) for n in (
            "max_seq_len", "gdn_conv_dim", "gdn_value_dim", "gdn_num_v_heads", "gdn_num_k_heads",
            "gdn_head_dim", "gdn_conv_kernel", "mla_kv_lora_rank", "mla_qk_nope_head_dim",
            "mla_qk_rope_head_dim", "mla_v_head_dim", "max_chunk")]


def _declare(lib):
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ffn_int4_last_error.restype = ctypes.c_char_p
    lib.ffn_int4_last_error.argtypes = []
    sigs = {
        "ffn_int4_abi_version": [],
        "ffn_int4_device_status": [ctypes.POINTER(ci), ctypes.POINTER(ci)],
        "ffn_int4_set_fused": [ci],
        "ffn_int4_set_decode_kernel": [ci],
        "ffn_int4_set_launch_overlap": [ci],
        "ffn_int4_set_batched_kernel": [ci],
        "ffn_gemm_int4_bf16": [vp, vp, vp, vp, ci, ci, ci, ci, vp],
        "ffn_silu_mul_packed": [vp, vp, ci, ci, vp],
        "ffn_gemma_rms_norm": [vp, vp, vp, ci, ci, cf, vp],
        "ffn_residual_add": [vp, vp, ci, vp],
        "ffn_dequantize_int4": [vp, vp, vp, ci, ci, vp, vp],
        "ffn_forward_mlp": [vp, vp, vp, vp, vp, ctypes.POINTER(MlpWeights), ci, ctypes.POINTER(ModelDims)],
        "ffn_forward_mlp_prepared": [vp, vp, vp, vp, vp, ctypes.POINTER(MlpWeights), ci,
                                     ctypes.POINTER(ModelDims)],
        "ffn_forward_mlp_prepared_noalloc": [vp, vp, vp, ctypes.POINTER(MlpWeights), ci, ctypes.POINTER(ModelDims)],
        "ffn_tp_create": [ctypes.POINTER(vp), ci, ci, ci, ci],
        "ffn_tp_export": [vp, vp],
        "ffn_tp_connect": [vp, vp],
        "ffn_tp_connect_local": [ctypes.POINTER(vp), ci],
        "ffn_tp_destroy": [vp],
        "ffn_forward_mlp_tp": [vp, vp, vp, vp, vp, ctypes.POINTER(MlpWeights), ci, ctypes.POINTER(ModelDims), vp],
        "ffn_decode_stack": [vp, vp, vp, vp, vp, ctypes.POINTER(MlpWeights), ci, ci, ctypes.POINTER(ModelDims)],
        "ffn_sha256_hex": [vp, ctypes.c_size_t, vp],
        "ffn_quant_manifest_parse": [ctypes.c_char_p, ctypes.POINTER(vp)],
        "ffn_quant_manifest_counts": [vp] + [ctypes.POINTER(ci)] * 4,
        "ffn_quant_manifest_find_entry": [vp, ci, ctypes.c_char_p],
        "ffn_quant_manifest_find_pair": [vp, ctypes.c_char_p, ci],
        "ffn_quant_manifest_entry_shape": [vp, ci] + [ctypes.POINTER(ctypes.c_longlong)] * 3 + [ctypes.POINTER(ci)],
        "ffn_quant_manifest_pair_shape": [vp, ci] + [ctypes.POINTER(ctypes.c_longlong)] * 3,
        "ffn_quant_artifact_read": [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_longlong,
                                    ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(vp),
                                    ctypes.POINTER(ctypes.c_size_t)],
        "ffn_shard_view": [ci, ctypes.c_longlong, ctypes.c_longlong, ci, ci, ctypes.POINTER(ctypes.c_longlong)],
        "ffn_load_quantized_ffn": [ctypes.c_char_p, ci, ci, ci, ci, ci, ctypes.POINTER(vp)],
        "ffn_load_quantized_ffn_ranks": [ctypes.c_char_p, ci, ci, ci, ci, ctypes.POINTER(ci), ctypes.POINTER(vp)],
        "ffn_quantized_ffn_layer": [vp, ci, ctypes.POINTER(MlpWeights)],
        "ffn_quantized_ffn_free": [vp],
        "ffn_quantized_ffn_prepare_decode": [vp],
        "test_gemm_int4": [vp, vp, vp, vp, ci, ci, ci, ci],
        "test_silu_mul_packed": [vp, vp, ci, ci],
        "test_norm": [vp, vp, vp, ci, ci],
        "test_silu_mul": [vp, vp, ci],
        "test_residual_norm": [vp, vp, vp, vp, ci, ci, ctypes.c_float, ci],
        "ffn_residual_norm": [vp, vp, vp, vp, ci, ci, ctypes.c_float, ci, vp],
        "ffn_silu_mul": [vp, vp, ci, vp],
        "ffn_quantize_int4": [vp, vp, vp, ctypes.c_longlong, ctypes.c_longlong, vp],
        "ffn_int4_describe_plan": [ci, ci, ci, ci, ci, ctypes.c_char_p, ctypes.c_size_t],
        "ffn_convert_checkpoint": [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_char_p), ci, ci],
        "ffn_json_reencode": [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t],
        "ffn_verify_sidecar": [ctypes.c_char_p, ci, ctypes.c_char_p, ctypes.c_size_t],
        "ffn_int4_noalloc_status": [ctypes.POINTER(ci), ctypes.POINTER(ci)],
        "ffn_decode_layer_prepare": [ctypes.POINTER(MlpWeights), ctypes.POINTER(ModelDims), vp],
        "ffn_decode_layer_release": [ctypes.POINTER(MlpWeights)],
        "ffn_decode_layer_is_prepared": [ctypes.POINTER(MlpWeights)],
        "ffn_int4_describe_kmajor_plan": [ci, ci, ci, ci, ci, ctypes.c_char_p, ctypes.c_size_t],
        "ffn_int4_describe_gemm_plan": [ci, ci, ci, ci, ci, ctypes.c_char_p, ctypes.c_size_t],
        "ffn_forward_mlp_host": [vp, vp, vp, vp, vp, vp, ctypes.POINTER(MlpWeights), ci, ctypes.POINTER(ModelDims)],
        "ffn_tp_allreduce_sum": [vp, vp, vp, ctypes.c_size_t, ci],
        "ffn_allreduce_sum": [ctypes.POINTER(vp), ctypes.POINTER(vp), ci, ctypes.POINTER(vp), ctypes.c_size_t, ci],
    }
    lib.ffn_tp_exchange_tag.argtypes = [ctypes.c_uint]
    lib.ffn_tp_exchange_tag.restype = ctypes.c_uint
    lib.ffn_int4_numerical_policy.argtypes = []
    lib.ffn_int4_numerical_policy.restype = ctypes.c_char_p
    lib.ffn_quant_manifest_free.argtypes = [vp]
    lib.ffn_quant_manifest_free.restype = None
    lib.ffn_host_free.argtypes = [vp]
    lib.ffn_host_free.restype = None
    lib.ffn_int4_tile_order_offset.argtypes = [ci, ci, ci]
    lib.ffn_int4_tile_order_offset.restype = ctypes.c_longlong
    lib.ffn_int4_debug_trace.argtypes = [vp]
    lib.ffn_int4_debug_trace.restype = None
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ci
    return lib


def load():
    """The loaded library.  Raises LibraryMissing if it was never built (run
    ``python haskell-infer-demo_b200/build.py``); there is no fallback implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} is missing: build it with `python haskell-infer-demo_b200/build.py`; "
                "this package has no CPU or PyTorch fallback")
        _lib = _declare(ctypes.CDLL(LIB_PATH))
    return _lib


def device_status():
    """Synchronise and raise FfnError if a fused kernel gave up on a bounded wait."""
    where, cta = ctypes.c_int(0), ctypes.c_int(0)
    return check(load().ffn_int4_device_status(ctypes.byref(where), ctypes.byref(cta)))


def check(status):
    """Raise FfnError for a negative status, carrying the library's message."""
    if status != 0:
        raise FfnError(status, load().ffn_int4_last_error().decode("utf-8", "replace"))
    return status
