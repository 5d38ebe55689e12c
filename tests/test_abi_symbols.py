"""CPU-only checks of the shipped library: it builds, loads, and exports every function that
include/ffn_int4.h declares.  No compute entry point is called here (there is no GPU)."""
import os
import re

from haskell_infer_demo_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for header in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"^\s*(?:const\s+)?(?:int|char|void|size_t|long long|unsigned)\s*\*?\s*(\w+)\s*\(",
                            text, flags=re.M)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_functions()
    assert "ffn_gemm_int4_bf16" in names and "ffn_forward_mlp" in names and "test_gemm_int4" in names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"
    assert lib.ffn_int4_abi_version() == 1


def test_argument_refusals_need_no_gpu():
    """Validation happens before any CUDA call, in the reference's order
    (csrc/kernels/gemm_quant.cu:208-224), and reports through status + last error."""
    lib = L.load()
    assert lib.ffn_gemm_int4_bf16(16, 16, 16, 16, -1, 8, 128, 128, None) == -4
    assert b"negative extent" in lib.ffn_int4_last_error()
    assert lib.ffn_gemm_int4_bf16(16, 16, 16, 16, 0, 8, 128, 128, None) == 0      # M == 0: no-op
    assert lib.ffn_gemm_int4_bf16(None, 16, 16, 16, 1, 8, 128, 128, None) == -4
    assert b"null buffer" in lib.ffn_int4_last_error()
    assert lib.ffn_gemm_int4_bf16(16, 16, 16, 16, 1, 128, 192, 128, None) == -4    # 1.5 groups
    assert b"not a whole number" in lib.ffn_int4_last_error()
    assert lib.ffn_gemm_int4_bf16(16, 16, 16, 16, 1, 128, 128, 64, None) == -4     # foreign group
    assert lib.ffn_silu_mul_packed(16, 16, -1, 4, None) == -4
    assert lib.ffn_silu_mul_packed(None, None, 0, 4, None) == 0
    assert lib.ffn_residual_add(None, None, 4, None) == -4
    assert lib.test_gemm_int4(16, 16, 16, 16, 1, 128, 192, 128) != 0              # bridge refuses too


def test_struct_mirrors_match_header_sizes():
    import ctypes
    assert ctypes.sizeof(L.MlpWeights) == 8 * 8 + 8      # eight pointers + int, padded
    assert ctypes.sizeof(L.ModelDims) == 25 * 4


def test_new_entries_validate_before_any_cuda_call():
    lib = L.load()
    assert lib.ffn_residual_norm(16, 16, 16, 16, 0, 1, 1e-6, 1, None) == -4
    assert b"invalid shape or epsilon" in lib.ffn_int4_last_error()
    assert lib.ffn_residual_norm(16, None, 16, 16, 128, 1, 1e-6, 1, None) == -4
    assert b"null buffer" in lib.ffn_int4_last_error()
    assert lib.ffn_residual_norm(None, None, None, None, 128, 0, 1e-6, 0, None) == 0     # no rows: nothing to do
    assert lib.ffn_silu_mul(16, 16, -1, None) == -4
    assert lib.ffn_silu_mul(16, 18, 16, None) == -4                                     # misaligned gate
    assert lib.ffn_quantize_int4(16, 16, 16, 8, 192, None) == -4
    assert b"whole number" in lib.ffn_int4_last_error()
    assert lib.ffn_quantize_int4(16, 16, 16, 12, 128, None) == -4
    assert b"8-row tile" in lib.ffn_int4_last_error()
    assert lib.ffn_quantize_int4(None, 16, 16, 8, 128, None) == -4


def test_compute_entries_fail_loudly_without_a_gpu():
    """There is no CPU fallback: on a machine without a CUDA device every compute entry point returns
    an error status with a message, it never computes on the host."""
    import ctypes

    import numpy as np
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("this machine has a GPU")
    lib = L.load()
    buf = np.zeros(4096, np.uint16)
    p = buf.ctypes.data
    assert lib.ffn_gemm_int4_bf16(p, p, p, p, 1, 8, 128, 128, None) < 0 and lib.ffn_int4_last_error()
    assert lib.ffn_quantize_int4(p, p, p, 8, 128, None) < 0 and lib.ffn_int4_last_error()
    assert lib.test_gemm_int4(p, p, p, p, 1, 8, 128, 128) != 0
    handle = ctypes.c_void_p()
    assert lib.ffn_tp_create(ctypes.byref(handle), 2, 0, 1024, 2) < 0
    assert b"CUDA" in lib.ffn_int4_last_error()
    w, d = L.MlpWeights(), L.ModelDims()
    w.gate_up_i4 = w.gate_up_i4_scales = w.down_i4 = w.down_i4_scales = p
    w.i4_group = 128
    d.hidden_size, d.intermediate_size, d.max_chunk, d.rms_eps = 128, 128, 128, 1e-6
    assert lib.ffn_forward_mlp_prepared(None, None, p, p, p, ctypes.byref(w), 1, ctypes.byref(d)) < 0
    assert lib.ffn_int4_last_error()
    assert lib.ffn_forward_mlp_prepared_noalloc(None, p, p, ctypes.byref(w), 1, ctypes.byref(d)) < 0
    assert lib.ffn_int4_noalloc_status(None, None) < 0 and lib.ffn_int4_last_error()
    assert lib.ffn_forward_mlp_host(None, None, p, p, p, p, ctypes.byref(w), 1, ctypes.byref(d)) < 0


def test_exchange_tag_is_never_zero_across_the_counter_wrap():
    """A zero tag means "nobody wrote this word since the buffer was cleared", so no call number may
    map to it - also not the last value of the 32-bit call counter."""
    lib = L.load()
    for call in (0, 1, 2, 0x7FFFFFFF, 0x80000000, 0xFFFFFFFD, 0xFFFFFFFE, 0xFFFFFFFF):
        assert lib.ffn_tp_exchange_tag(call) != 0
    # consecutive calls use the two slot parities alternately, so equal tags on calls n and n+1 are harmless;
    # calls n and n+2 (the same slots) must differ
    for call in (0, 5, 0xFFFFFFFD, 0xFFFFFFFE, 0xFFFFFFFF):
        assert lib.ffn_tp_exchange_tag(call) != lib.ffn_tp_exchange_tag((call + 2) & 0xFFFFFFFF)


def test_new_host_side_validation_and_identity():
    import ctypes
    lib = L.load()
    fields = lib.ffn_int4_numerical_policy().decode()
    import json
    parsed = json.loads("{" + fields + "}")
    assert list(parsed) == sorted(parsed)                     # sorted keys, as the manifest emitter writes them
    assert parsed["weight_quantization"] == "int4_symmetric_group_bf16_scale_decode_only"   # csrc/manifest.c:433-434
    assert lib.ffn_tp_allreduce_sum(None, None, None, 4, 2) == -4
    assert lib.ffn_allreduce_sum(None, None, 2, None, 4, 2) == -4
    assert lib.ffn_allreduce_sum(None, None, 1, None, 4, 2) == -4      # null arrays are refused before the count is looked at
    w, d = L.MlpWeights(), L.ModelDims()
    assert lib.ffn_forward_mlp_host(None, None, None, None, None, None, ctypes.byref(w), 1, ctypes.byref(d)) == -4
    buf = ctypes.create_string_buffer(512)
    assert lib.ffn_int4_describe_gemm_plan(1, 4096, 5120, 148, 232448, buf, 512) == 0 and b"stream_gemv" in buf.value
    assert lib.ffn_int4_describe_gemm_plan(1, 4100, 5120, 148, 232448, buf, 512) == 0 and b"generic" in buf.value   # N % 8
    assert lib.ffn_int4_describe_gemm_plan(2, 4096, 34816, 148, 232448, buf, 512) == 0 and b"generic" in buf.value  # two rows: K <= 17408
    assert lib.ffn_int4_describe_gemm_plan(1, 4096, 192, 148, 232448, buf, 512) == -4


def test_header_conforms_to_the_reference_headers_where_a_checkout_exists():
    """Compile-only: include/ffn_int4.h against the reference's layers.h / engine.h (field offsets of
    both struct mirrors, status codes, prototypes), as the reference's engine stub includes engine.h so
    that drift breaks the build (tests/generation_engine_stub.c:1-12)."""
    import subprocess
    import sys

    import pytest
    sys.path.insert(0, ROOT)
    from __graft_entry__ import reference_checkout
    ref = reference_checkout()
    if not ref:
        pytest.skip("no reference checkout on this machine")
    obj = os.path.join(ROOT, "oracle", "_ref", "abi_conformance.o")
    if os.path.exists(obj):
        os.remove(obj)
    proc = subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), f"REFERENCE={ref}", "_ref/abi_conformance.o"],
                          capture_output=True, text=True)
    assert proc.returncode == 0 and os.path.exists(obj), proc.stdout + proc.stderr


def test_kernel_switches_query_set_and_restore_without_a_gpu():
    """The A/B switches are plain host state: a value outside their range queries, a set returns the
    previous setting, and the defaults are the measured-faster kernels."""
    lib = L.load()
    for name, default, other in (("ffn_int4_set_decode_kernel", 1, 0), ("ffn_int4_set_batched_kernel", 2, 1),
                                 ("ffn_int4_set_launch_overlap", 1, 0)):
        fn = getattr(lib, name)
        assert fn(-1) == default, name
        assert fn(other) == default and fn(-1) == other, name
        assert fn(default) == other and fn(-1) == default, name
    assert lib.ffn_quantized_ffn_prepare_decode(None) == -4 and b"null handle" in lib.ffn_int4_last_error()
