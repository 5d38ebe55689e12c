"""GPU parity of the INT4 GEMM entry points through the C ABI, shaped like the reference's own
kernel gate (tests/test_quantization_kernel.py): same shapes, token counts, data recipe, float64
dequantized reference and acceptance numbers (max_rel <= 8e-3, rms_rel <= 4e-3, K=192 refused)."""
import ctypes

import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200 import ops
from oracle import ffn_oracle as o
from gpu_util import dev_bits, dev_u8, host_f32

pytestmark = pytest.mark.gpu

SHAPES = [(256, 128), (1024, 256), (4096, 5120)]
M_VALUES = [1, 2, 8, 64]


def gate_weights(rng, n, k):
    w = (rng.randn(n, k) * 0.05).astype(np.float32)
    w *= (1.0 + 0.5 * rng.rand(n, k // 128).astype(np.float32)).repeat(128, axis=1)
    return w


@pytest.mark.parametrize("n,k", SHAPES)
def test_kernel_gate_host_pointers(cuda, n, k):
    """test_gemm_int4 with HOST numpy pointers, exactly as the reference's gate calls its bridge
    (tests/test_quantization_kernel.py:118-123)."""
    lib = L.load()
    rng = np.random.RandomState(11)
    w = gate_weights(rng, n, k)
    packed, scales = o.quantize(w)
    deq = o.dequantize(packed, scales)
    for m in M_VALUES:
        x = (rng.randn(m, k) * 0.5).astype(np.float32)
        a_bits = o.bf16_bits(x)
        ref = o.bf16_to_f32(a_bits).astype(np.float64) @ deq.astype(np.float64).T
        out = np.empty((m, n), np.uint16)
        st = lib.test_gemm_int4(out.ctypes.data, a_bits.ctypes.data, packed.ctypes.data,
                                scales.ctypes.data, m, n, k, 128)
        assert st == 0, lib.ffn_int4_last_error()
        got = o.bf16_to_f32(out).astype(np.float64)
        err = np.abs(got - ref)
        scale = max(float(np.abs(ref).max()), 1e-9)
        assert err.max() / scale <= 8e-3, (m, n, k)
        assert np.sqrt((err ** 2).mean()) / scale <= 4e-3, (m, n, k)


def test_kernel_gate_refuses_partial_group(cuda):
    lib = L.load()
    n, k = 128, 192
    bad = np.zeros(n * k // 2, np.uint8)
    sc = np.zeros(n, np.uint16)
    out = np.zeros((1, n), np.uint16)
    assert lib.test_gemm_int4(out.ctypes.data, out.ctypes.data, bad.ctypes.data, sc.ctypes.data,
                              1, n, k, 128) != 0


@pytest.mark.parametrize("n,k", [(8, 128), (1024, 256), (3072, 1024), (1024, 3072)])
def test_dequantized_weights_bit_exact(cuda, n, k):
    """The kernels' unpack routine reproduces linear_dequantize_int4 bit for bit."""
    rng = np.random.default_rng(n + k)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    w[0, :128] = 0.0                       # zero group -> scale 1.0
    w[1, 0], w[1, 1] = 0.7000001, -0.7000001
    packed, scales = o.quantize(w)
    want = o.dequantize(packed, scales)
    got, bad = ops.dequantize_int4(dev_u8(packed, cuda), dev_bits(scales, cuda))
    assert bad == 0
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    packed[2, 3] = 0x80                    # a reserved code is counted, as the reader refuses it
    _, bad = ops.dequantize_int4(dev_u8(packed, cuda), dev_bits(scales, cuda))
    assert bad == 1


@pytest.mark.parametrize("m", [1, 3, 5, 16])
def test_gemm_device_pointers_and_ragged_m(cuda, m):
    rng = np.random.default_rng(m)
    n, k = 264, 384                        # N not a multiple of the block's 32 rows
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    packed, scales = o.quantize(w)
    x = o.bf16_round(rng.standard_normal((m, k), dtype=np.float32))
    ref = o.matmul_packed_f64(x, packed, scales)
    out = ops.gemm_int4_bf16(dev_bits(o.bf16_bits(x), cuda), dev_u8(packed, cuda), dev_bits(scales, cuda))
    torch.cuda.synchronize()
    err = np.abs(host_f32(out).astype(np.float64) - ref)
    assert err.max() / np.abs(ref).max() <= 8e-3


def test_silu_norm_residual(cuda):
    rng = np.random.default_rng(3)
    t, i = 3, 1000
    pk = o.bf16_round(rng.standard_normal((t, 2 * i), dtype=np.float32) * 3)
    got = host_f32(ops.kernel_silu_mul_packed(dev_bits(o.bf16_bits(pk), cuda)))
    want = o.silu_mul(pk[:, :i], pk[:, i:])
    # device __expf vs numpy exp: at most one BF16 ulp apart (tests/test_library_ops.py:97-125)
    assert np.abs(got - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
    for cols in (128, 256, 5120):          # tests/test_library_ops.py:48-60
        x = o.bf16_round(rng.standard_normal((4, cols), dtype=np.float32))
        x[1] = 0.0
        x[2] *= 1e-4
        x = o.bf16_round(x)
        wn = o.bf16_round(rng.standard_normal(cols, dtype=np.float32) * np.float32(0.1))
        got = host_f32(ops.kernel_gemma_rms_norm(dev_bits(o.bf16_bits(x), cuda), dev_bits(o.bf16_bits(wn), cuda)))
        want = o.gemma_rmsnorm(x, wn)
        assert np.allclose(got, want, atol=1e-3, rtol=8e-3)
    h = o.bf16_round(rng.standard_normal((2, 512), dtype=np.float32))
    y = o.bf16_round(rng.standard_normal((2, 512), dtype=np.float32))
    dst = dev_bits(o.bf16_bits(h), cuda).clone()
    ops.kernel_residual_add(dst, dev_bits(o.bf16_bits(y), cuda))
    assert np.array_equal(host_f32(dst), o.residual_add(h, y))


@pytest.mark.parametrize("rows,hidden", [(1, 256), (4, 256), (3, 100), (2, 5000), (2, 5120), (1, 9000)])
@pytest.mark.parametrize("gemma", [0, 1])
def test_residual_norm_rounding_rule(cuda, rows, hidden, gemma):
    """The reference's gate for the fused residual + norm (tests/test_residual_norm.py:30-150), through
    the same bridge entry with host pointers: the updated residual is bitwise bf16(r + s); the norm is
    within 8e-3 of the expression evaluated on the ROUNDED residual and no further from it than from
    the one evaluated on the unrounded sum.  Shapes are the reference's plus the 27B row and one row
    longer than the kernel keeps in registers."""
    rng = np.random.default_rng(11 + rows * 7 + hidden + gemma)
    res = o.bf16_round(rng.standard_normal((rows, hidden), dtype=np.float32) * np.float32(1.5))
    sub = o.bf16_round(rng.standard_normal((rows, hidden), dtype=np.float32) * np.float32(1.5))
    w = o.bf16_round(rng.standard_normal(hidden, dtype=np.float32) * np.float32(0.1))
    kept = o.bf16_bits(res).copy()
    normed = np.zeros((rows, hidden), np.uint16)
    sub_bits, w_bits = o.bf16_bits(sub), o.bf16_bits(w)
    st = L.load().test_residual_norm(normed.ctypes.data, kept.ctypes.data, sub_bits.ctypes.data, w_bits.ctypes.data,
                                     hidden, rows, 1e-6, gemma)
    assert st == 0
    want_r = o.residual_add(res, sub)
    assert np.array_equal(o.bf16_to_f32(kept), want_r)

    def norm_of(total):
        t64 = total.astype(np.float64)
        inv = 1.0 / np.sqrt((t64 * t64).mean(axis=-1, keepdims=True) + 1e-6)
        return o.bf16_round((t64 * inv * (w.astype(np.float64) + gemma)).astype(np.float32))
    got = o.bf16_to_f32(normed)
    want = norm_of(want_r)
    plain = norm_of(res.astype(np.float32) + sub.astype(np.float32))
    assert np.abs(got - want).max() / max(np.abs(want).max(), 1e-6) <= 8e-3
    assert np.abs(got - want).mean() <= np.abs(got - plain).mean()


def test_residual_norm_and_silu_mul_refusals(cuda):
    lib = L.load()
    buf = torch.zeros(64, dtype=torch.bfloat16, device=cuda)
    p = buf.data_ptr()
    assert lib.ffn_residual_norm(p, p, p, p, 0, 1, 1e-6, 1, None) == -4       # invalid shape
    assert lib.ffn_residual_norm(p, p, p, p, 16, 1, 0.0, 1, None) == -4       # invalid epsilon
    assert lib.ffn_residual_norm(p, None, p, p, 16, 1, 1e-6, 1, None) == -4   # null buffer
    assert lib.ffn_residual_norm(p, p, p, p, 16, 0, 1e-6, 1, None) == 0                     # no rows: nothing to do
    assert lib.ffn_silu_mul(p, p, -1, None) == -4
    assert lib.ffn_silu_mul(p, p + 2, 16, None) == -4                         # misaligned
    assert lib.ffn_silu_mul(p, p, 12, None) == -4                             # n >= 8 must be a multiple of 8
    assert lib.ffn_silu_mul(p, p, 0, None) == 0


@pytest.mark.parametrize("n", [4, 8, 1024, 17408])
def test_silu_mul_pair(cuda, n):
    """kernel_silu_mul's contract (csrc/kernels/silu.cu:29-52): contiguous [gate[n] | up[n]], FP32 SiLU*up,
    one rounding; checked as tests/test_library_ops.py does (within one BF16 step of the FP64 value)."""
    rng = np.random.default_rng(n)
    gu = o.bf16_round(rng.standard_normal(2 * n, dtype=np.float32) * 3)
    bits = o.bf16_bits(gu)
    out = np.zeros(n, np.uint16)
    assert L.load().test_silu_mul(out.ctypes.data, bits.ctypes.data, n) == 0
    want = o.silu_mul(gu[:n], gu[n:])
    assert np.abs(o.bf16_to_f32(out) - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
