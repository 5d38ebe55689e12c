"""CPU oracle for the INT4 dense-FFN decode path.  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the bench's CPU-baseline legs may import this module; the
shipped package never does.  It restates, on the CPU, the arithmetic the reference performs for

    y = W_down . ( SiLU(W_gate . n) * (W_up . n) ),   n = GemmaRMSNorm(h)   (optional)

with the reference's rounding points, in the order of ``mlp_from_normed``
(csrc/kernels/layers.cu:104-147):

1. ``W = float(code) * float(scale)``          - linear_dequantize_int4, csrc/linear_weight.cpp:178-216
2. ``g, u = bf16(sum_k W[n,k] * x[k])``        - gemv_int4_kernel rounds its output to BF16,
                                                 csrc/kernels/gemm_quant.cu:199; accumulation here is
                                                 FP64 like tests/test_quantization_kernel.py:115
3. ``a = bf16(g / (1 + exp(-g)) * u)``         - silu_mul_packed_kernel, csrc/kernels/silu.cu:61-74
4. ``y = bf16(sum_i W_down[h,i] * a[i])``      - same GEMV; under tensor parallelism the oracle is
                                                 still this whole-I sum (the TP=1 value)
5. ``n = bf16(x * rsqrt(mean(x^2)+eps) * (1+w))`` - Gemma RMSNorm as the reference's tests define it,
                                                 tests/test_library_ops.py:55-57, tests/kernels/test_norm.cu:14-32
6. ``h = bf16(f32(h) + f32(y))``               - residual_add_kernel, csrc/kernels/gdn_norm.cu:121-129

Parity is PINNED: the format half is checked against the reference's known-answer vectors and,
where the reference sources exist, bit-for-bit against its compiled quantizer (oracle/_ref).
The FFN chain is a composition of those pieces (the reference has no single CPU function for it).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

GROUP = 128
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle_int4.so")
        if not os.path.exists(path):
            subprocess.run(["make", "-C", _HERE, "liboracle_int4.so"], check=True,
                           capture_output=True)
        lib = ctypes.CDLL(path)
        lib.orc_quantize.argtypes = [ctypes.c_longlong, ctypes.c_longlong] + [ctypes.c_void_p] * 3
        lib.orc_dequantize.argtypes = [ctypes.c_longlong, ctypes.c_longlong] + [ctypes.c_void_p] * 3
        lib.orc_matmul_f64.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong] + \
            [ctypes.c_void_p] * 3
        lib.orc_matmul_f64.restype = None
        lib.orc_matmul_packed_f64.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong] + \
            [ctypes.c_void_p] * 4
        lib.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        lib.orc_f32_to_bf16.restype = ctypes.c_uint16
        lib.orc_bf16_to_f32.argtypes = [ctypes.c_uint16]
        lib.orc_bf16_to_f32.restype = ctypes.c_float
        lib.orc_packed_code.argtypes = [ctypes.c_void_p] + [ctypes.c_longlong] * 3
        lib.orc_layout.argtypes = [ctypes.c_longlong] * 3 + [ctypes.c_void_p] * 2
        _LIB = lib
    return _LIB


def ref_lib(name="libref_linear_weight.so"):
    """The reference's own code compiled by oracle/Makefile, or None when it was never built."""
    path = os.path.join(_HERE, "_ref", name)
    return ctypes.CDLL(path) if os.path.exists(path) else None


# ---------------------------------------------------------------------------------------------
# BF16 helpers (round to nearest even, csrc/linear_weight.cpp:34-51)
# ---------------------------------------------------------------------------------------------
def bf16_bits(values) -> np.ndarray:
    """FP32 array -> BF16 bit patterns (uint16)."""
    u = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFFFFFF
    return (u >> 16).astype(np.uint16)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(values) -> np.ndarray:
    """FP32/FP64 array -> FP32 array holding BF16-representable values."""
    return bf16_to_f32(bf16_bits(np.asarray(values, dtype=np.float32)))


# ---------------------------------------------------------------------------------------------
# The format
# ---------------------------------------------------------------------------------------------
def quantize(weights: np.ndarray):
    """FP32 [N, K] -> (packed u8 [N, K/2], scales u16 [N, K/128]).  Raises on refusal."""
    w = np.ascontiguousarray(weights, dtype=np.float32)
    n, k = w.shape
    if n <= 0 or k <= 0 or k % GROUP or n % 8:
        raise ValueError(f"the INT4 format cannot hold [{n}, {k}]")
    packed = np.zeros((n, k // 2), dtype=np.uint8)
    scales = np.zeros((n, k // GROUP), dtype=np.uint16)
    status = _lib().orc_quantize(n, k, w.ctypes.data, packed.ctypes.data, scales.ctypes.data)
    if status != 0:
        raise ValueError(f"orc_quantize refused the tensor (status {status})")
    return packed, scales


def dequantize(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """(packed [N, K/2], scales [N, K/128]) -> FP32 [N, K]; exact code*scale products."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    n, kb = packed.shape
    k = kb * 2
    out = np.empty((n, k), dtype=np.float32)
    status = _lib().orc_dequantize(n, k, packed.ctypes.data, scales.ctypes.data, out.ctypes.data)
    if status != 0:
        raise ValueError(f"orc_dequantize refused the artifact (status {status})")
    return out


def dequantize_numpy(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """The same definition in pure numpy (a second statement, used to cross-check the C one);
    mirrors dequantize_independent in tests/test_quantization_kernel.py:60-69."""
    n, kb = packed.shape
    lo = (packed & 0x0F).astype(np.int32)
    hi = (packed >> 4).astype(np.int32)
    codes = np.empty((n, kb * 2), dtype=np.int32)
    codes[:, 0::2] = np.where(lo >= 8, lo - 16, lo)
    codes[:, 1::2] = np.where(hi >= 8, hi - 16, hi)
    s = bf16_to_f32(scales).reshape(n, -1)
    return codes.astype(np.float32) * np.repeat(s, GROUP, axis=1)


def matmul_f64(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    """a [M, K] FP32, w [N, K] FP32 -> FP64 [M, N] with FP64 accumulation."""
    return a.astype(np.float64) @ w.astype(np.float64).T


def matmul_packed_f64(a: np.ndarray, packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """a [M, K] FP32 times the packed weight [N, K], FP64 accumulation, no FP32 weight copy."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    m, k = a.shape
    n = packed.shape[0]
    out = np.empty((m, n), dtype=np.float64)
    status = _lib().orc_matmul_packed_f64(m, n, k, a.ctypes.data, packed.ctypes.data,
                                          scales.ctypes.data, out.ctypes.data)
    if status != 0:
        raise ValueError("orc_matmul_packed_f64 refused the shape")
    return out


# ---------------------------------------------------------------------------------------------
# Tensor-parallel slicing (engine_load_quantized_ffn, csrc/engine.cu:2308-2401; shard views
# csrc/model_desc.c:609-626).  Scales are the global ones the slice selects, never re-derived.
# ---------------------------------------------------------------------------------------------
def shard_out_dim(rows: int, tp: int, rank: int):
    if rows % tp:
        raise ValueError(f"tp_size {tp} does not divide {rows} rows")
    per = rows // tp
    return per * rank, per


def shard_in_dim(cols: int, tp: int, rank: int):
    if cols % tp:
        raise ValueError(f"tp_size {tp} does not divide {cols} columns")
    per = cols // tp
    return per * rank, per


def slice_rank(gate_up_packed, gate_up_scales, down_packed, down_scales, tp: int, rank: int):
    """One rank's operands from the whole artifacts.

    gate_up is the [2I, H] pair (gate rows then up rows); the rank keeps gate rows and up rows
    [r*I/R, (r+1)*I/R).  down is [H, I]; the rank keeps columns [r*I/R, (r+1)*I/R), which must
    start on a group boundary (csrc/engine.cu:2316-2322).
    """
    two_i, hb = gate_up_packed.shape
    inter = two_i // 2
    row_off, rows = shard_out_dim(inter, tp, rank)
    col_off, cols = shard_in_dim(down_packed.shape[1] * 2, tp, rank)
    if col_off % GROUP or cols % GROUP:
        raise ValueError("splits K at a non-group boundary, which cannot retain the global scales")
    gu_p = np.concatenate([gate_up_packed[row_off:row_off + rows],
                           gate_up_packed[inter + row_off:inter + row_off + rows]], axis=0)
    gu_s = np.concatenate([gate_up_scales[row_off:row_off + rows],
                           gate_up_scales[inter + row_off:inter + row_off + rows]], axis=0)
    d_p = down_packed[:, col_off // 2:(col_off + cols) // 2]
    d_s = down_scales[:, col_off // GROUP:(col_off + cols) // GROUP]
    return (np.ascontiguousarray(gu_p), np.ascontiguousarray(gu_s),
            np.ascontiguousarray(d_p), np.ascontiguousarray(d_s))


# ---------------------------------------------------------------------------------------------
# The FFN chain
# ---------------------------------------------------------------------------------------------
def silu_mul(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """bf16(g/(1+exp(-g)) * u) on BF16-valued FP32 inputs, FP32 math (csrc/kernels/silu.cu:70-72)."""
    g = g.astype(np.float32)
    u = u.astype(np.float32)
    return bf16_round((g / (np.float32(1.0) + np.exp(-g))) * u)


def gemma_rmsnorm(h: np.ndarray, w_norm: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """bf16(x * rsqrt(mean(x^2) + eps) * (1 + w)); h [M, H] and w_norm [H] hold BF16 values."""
    x = h.astype(np.float64)
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return bf16_round((x * inv * (1.0 + w_norm.astype(np.float64))).astype(np.float32))


def residual_add(h: np.ndarray, y: np.ndarray) -> np.ndarray:
    return bf16_round(h.astype(np.float32) + y.astype(np.float32))


class Layer:
    """One quantized dense FFN layer: whole artifacts plus (optional) Gemma norm weight."""

    def __init__(self, gate_up_packed, gate_up_scales, down_packed, down_scales, w_norm=None):
        self.gate_up_packed = gate_up_packed
        self.gate_up_scales = gate_up_scales
        self.down_packed = down_packed
        self.down_scales = down_scales
        self.w_norm = w_norm  # FP32 array of BF16 values, or None
        self.inter = gate_up_packed.shape[0] // 2
        self.hidden = gate_up_packed.shape[1] * 2


def ffn(layer: Layer, x: np.ndarray, accumulate="f64", intermediates=False):
    """x [M, H] BF16-valued FP32 -> y [M, H] BF16-valued FP32 (steps 1-4 of the module doc).

    accumulate: "f64" (the gate's float64 matmul) or "f32" (an FP32-accumulating variant used
    only to measure how far two legitimate oracles drift apart on a deep stack).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    # many tokens: the same FP64 sums through BLAS on the dequantized weights (the C loop over the
    # packed bytes is single-threaded); a few tokens: straight from the packed bytes
    blas = accumulate == "f64" and x.shape[0] > 4
    if blas:
        gu = matmul_f64(x, dequantize(layer.gate_up_packed, layer.gate_up_scales))
    elif accumulate == "f64":
        gu = matmul_packed_f64(x, layer.gate_up_packed, layer.gate_up_scales)
    else:
        gu = x @ dequantize(layer.gate_up_packed, layer.gate_up_scales).T
    gu = bf16_round(gu.astype(np.float32))
    act = silu_mul(gu[:, :layer.inter], gu[:, layer.inter:])
    if blas:
        y = matmul_f64(act, dequantize(layer.down_packed, layer.down_scales))
    elif accumulate == "f64":
        y = matmul_packed_f64(act, layer.down_packed, layer.down_scales)
    else:
        y = act @ dequantize(layer.down_packed, layer.down_scales).T
    y = bf16_round(y.astype(np.float32))
    if intermediates:
        return y, gu, act
    return y


def ffn_reference_tp(layer: Layer, x: np.ndarray, tp: int) -> np.ndarray:
    """What the reference's own TP arithmetic produces: every rank rounds its down partial to
    BF16 (csrc/kernels/gemm_quant.cu:199) and the leader adds them one by one, rounding to BF16
    after every add (csrc/collective.cu:65-72, 182-192).  Reported for information only."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    total = None
    for r in range(tp):
        gu_p, gu_s, d_p, d_s = slice_rank(layer.gate_up_packed, layer.gate_up_scales,
                                          layer.down_packed, layer.down_scales, tp, r)
        gu = bf16_round(matmul_packed_f64(x, gu_p, gu_s).astype(np.float32))
        half = gu.shape[1] // 2
        act = silu_mul(gu[:, :half], gu[:, half:])
        part = bf16_round(matmul_packed_f64(act, d_p, d_s).astype(np.float32))
        total = part if total is None else bf16_round(total + part)
    return total


def stack(layers, h0: np.ndarray, accumulate="f64", teacher=None):
    """Config-4 stack: h <- h + FFN(GemmaRMSNorm(h)) per layer.  Returns the list of h after
    every layer (BF16-valued FP32).  With ``teacher`` (a list of per-layer inputs) every layer
    is fed teacher[l] instead of the running state."""
    h = np.ascontiguousarray(h0, dtype=np.float32)
    out = []
    for l, layer in enumerate(layers):
        src = h if teacher is None else teacher[l]
        n = gemma_rmsnorm(src, layer.w_norm)
        y = ffn(layer, n, accumulate=accumulate)
        h = residual_add(src, y)
        out.append(h)
    return out


# ---------------------------------------------------------------------------------------------
# Seeded synthetic configurations (stand-ins for the checkpoints the reference measures on)
# ---------------------------------------------------------------------------------------------
CONFIGS = {
    0: dict(hidden=1024, inter=3072, seed=0),
    1: dict(hidden=2560, inter=9728, seed=1),
    2: dict(hidden=5120, inter=17408, seed=2),
    3: dict(hidden=5120, inter=17408, seed=3),
    4: dict(hidden=5120, inter=17408, seed=4),
}


def draw_layer(rng: np.random.Generator, hidden: int, inter: int, with_norm: bool) -> Layer:
    """Draw order: W_gate [I,H], W_up [I,H], W_down [H,I] ~ N(0, 0.02) FP32, then w_norm [H] ~
    N(0, 0.1) rounded to BF16 when requested."""
    w_gate = rng.standard_normal((inter, hidden), dtype=np.float32) * np.float32(0.02)
    w_up = rng.standard_normal((inter, hidden), dtype=np.float32) * np.float32(0.02)
    w_down = rng.standard_normal((hidden, inter), dtype=np.float32) * np.float32(0.02)
    gp, gs = quantize(w_gate)
    up, us = quantize(w_up)
    dp, ds = quantize(w_down)
    w_norm = None
    if with_norm:
        w_norm = bf16_round(rng.standard_normal(hidden, dtype=np.float32) * np.float32(0.1))
    return Layer(np.concatenate([gp, up], axis=0), np.concatenate([gs, us], axis=0), dp, ds, w_norm)


def draw_config(hidden: int, inter: int, seed: int, tokens: int = 1, layers: int = 1,
                with_norm: bool = False):
    """Activations first ([M, H] ~ N(0,1) -> BF16), then the layers in order, all from
    numpy.random.default_rng(seed)."""
    rng = np.random.default_rng(seed)
    x = bf16_round(rng.standard_normal((tokens, hidden), dtype=np.float32))
    return x, [draw_layer(rng, hidden, inter, with_norm) for _ in range(layers)]


def compare(got: np.ndarray, want: np.ndarray):
    """(max-abs error, relative L2 error) between two BF16-valued arrays."""
    g = got.astype(np.float64).ravel()
    w = want.astype(np.float64).ravel()
    max_abs = float(np.abs(g - w).max()) if g.size else 0.0
    denom = float(np.sqrt((w * w).sum()))
    rel_l2 = float(np.sqrt(((g - w) ** 2).sum()) / denom) if denom > 0 else 0.0
    return max_abs, rel_l2
