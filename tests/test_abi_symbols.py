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
