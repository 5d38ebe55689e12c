"""Bit-exact pins of the hot kernels' own INT4 unpack, and the behaviour on non-finite inputs.

ffn_dequantize_int4 proves "dequantized weights are bit-exact" for the shape-generic kernel's unpack
only; the streaming kernel (dp4a on widened nibbles) and the tensor-core pair (lop3 to BF16 codes)
widen the codes in their own ways.  A single non-zero activation makes their arithmetic exact: every
output is then bf16(code * scale * activation), one product that FP32 holds without rounding, so the
outputs must equal the CPU statement of linear_dequantize_int4 (csrc/linear_weight.cpp:178-216)
times that activation BIT FOR BIT - which pins nibble order, sign extension and scale indexing of
every kernel on the path.
"""
import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200 import ops
from oracle import ffn_oracle as o
from gpu_util import dev_bf16, dev_bits, dev_u8, host_f32, upload_layer

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("n,k", [(264, 384), (1024, 256), (4096, 5120), (1024, 17408)])
@pytest.mark.parametrize("tokens", [1, 2, 8])
def test_one_hot_activation_gives_exact_dequantized_columns(cuda, n, k, tokens):
    """ffn_gemm_int4_bf16 with one-hot rows: one and two rows take the streaming kernel's
    single-matrix mode, eight the shape-generic kernel."""
    rng = np.random.default_rng(n * 7 + k + tokens)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    w[0, :128] = 0.0
    packed, scales = o.quantize(w)
    deq = o.dequantize(packed, scales)
    wd, sd = dev_u8(packed, cuda), dev_bits(scales, cuda)
    base = int(rng.integers(0, k - 8))
    for step in range(8):                       # eight neighbouring columns: every nibble position of a word
        x = np.zeros((tokens, k), np.float32)
        cols = [(base + step + 131 * m) % k for m in range(tokens)]
        vals = o.bf16_round(np.array([1.5, -0.3984375, 96.0, 2.0 ** -20, 1.0, -1.0, 0.0078125, 3.0][:tokens], np.float32))
        for m in range(tokens):
            x[m, cols[m]] = vals[m]
        out = ops.gemm_int4_bf16(dev_bf16(x, cuda), wd, sd)
        torch.cuda.synchronize()
        want = np.stack([o.bf16_bits(deq[:, cols[m]] * vals[m]) for m in range(tokens)])
        got = _bits(out)
        # -0.0 and +0.0 are the same value: compare zeros by value, everything else by bits
        same = (got == want) | (((got & 0x7FFF) == 0) & ((want & 0x7FFF) == 0))
        assert same.all(), f"N={n} K={k} M={tokens} column {cols}: {np.count_nonzero(~same)} outputs differ"
    L.device_status()


def _single_live_row_layer(hidden, inter, seed, live_rows):
    """Gate and up are zero except a few rows, so act has exactly those non-zero elements."""
    rng = np.random.default_rng(seed)
    wg = np.zeros((inter, hidden), np.float32)
    wu = np.zeros((inter, hidden), np.float32)
    for r in live_rows:
        wg[r] = rng.standard_normal(hidden, dtype=np.float32) * np.float32(0.05)
        wu[r] = rng.standard_normal(hidden, dtype=np.float32) * np.float32(0.05)
    wdn = rng.standard_normal((hidden, inter), dtype=np.float32) * np.float32(0.02)
    gp, gs = o.quantize(wg)
    up, us = o.quantize(wu)
    dp, ds = o.quantize(wdn)
    return o.Layer(np.concatenate([gp, up]), np.concatenate([gs, us]), dp, ds)


_LAYERS = {}


def _cached_layer(hidden, inter, row):
    if (hidden, inter, row) not in _LAYERS:
        _LAYERS.clear()                                   # one large layer at a time
        layer = _single_live_row_layer(hidden, inter, hidden, [row])
        _LAYERS[(hidden, inter, row)] = (layer, o.dequantize(layer.down_packed, layer.down_scales))
    return _LAYERS[(hidden, inter, row)]


@pytest.mark.parametrize("hidden,inter", [(1024, 3072), (5120, 17408)])
@pytest.mark.parametrize("tokens,kmajor", [(1, False), (2, False), (8, False), (16, False), (1, True), (2, True), (4, True),
                                           (1, "dp4a"), (2, "dp4a")])
def test_ffn_second_projection_is_exact_on_a_one_hot_act(cuda, hidden, inter, tokens, kmajor):
    """The whole FFN call (single-launch kernel for 1-2 tokens - row-major, or over the k-major copy of
    the down projection - and the tensor-core pair for 8 and 16) on a
    layer whose act has ONE non-zero element: y must equal bf16(dequantized down column * act) bit for
    bit, act being the value the device itself left in the workspace (SiLU uses the device's __expf,
    and the first projection rounds its sums, so act is only checked to be near the CPU chain's and
    then taken as given)."""
    live = [5 + 8 * 37]                                   # one row, not at a word boundary
    layer, deq_down = _cached_layer(hidden, inter, live[0])
    rng = np.random.default_rng(tokens)
    x = o.bf16_round(rng.standard_normal((tokens, hidden), dtype=np.float32))
    mlp = upload_layer(layer, cuda, prepare=bool(kmajor))
    ws = mlp.workspace(tokens)
    old = L.load().ffn_int4_set_decode_kernel(1 if kmajor == "dp4a" else 0)
    try:
        y = mlp.forward_mlp_prepared(dev_bf16(x, cuda), ws=ws)
        L.device_status()
    finally:
        L.load().ffn_int4_set_decode_kernel(old)
    act_dev = host_f32(ws[tokens * (hidden + 2 * inter):tokens * (hidden + 3 * inter)].view(tokens, inter))
    _, _, act_cpu = o.ffn(layer, x, intermediates=True)
    off = act_dev.copy()
    off[:, live] = 0.0
    assert not off.any(), "act must be zero wherever gate and up are zero"
    assert np.all(np.abs(act_dev - act_cpu) <= np.abs(act_cpu) * 2.0 ** -5 + 1e-30), "act is far from the CPU chain"
    want = np.stack([o.bf16_bits(deq_down[:, live[0]] * act_dev[m, live[0]]) for m in range(tokens)])
    got = _bits(y)
    same = (got == want) | (((got & 0x7FFF) == 0) & ((want & 0x7FFF) == 0))
    assert same.all(), f"H={hidden} I={inter} M={tokens}: {np.count_nonzero(~same)} outputs differ"


@pytest.mark.parametrize("tokens,kmajor", [(1, False), (2, False), (8, False), (1, True), (2, True), (3, True), (1, "dp4a"), (2, "dp4a")])
def test_ffn_first_projection_is_exact_on_a_one_hot_input(cuda, tokens, kmajor):
    """One-hot x: gate and up are single products, so act may differ from the CPU chain only through
    __expf (at most one BF16 ulp, and on few elements)."""
    hidden, inter = 1024, 3072
    _, layers = o.draw_config(hidden, inter, 17, tokens=tokens)
    layer = layers[0]
    mlp = upload_layer(layer, cuda, prepare=bool(kmajor))
    ws = mlp.workspace(tokens)
    old = L.load().ffn_int4_set_decode_kernel(1 if kmajor == "dp4a" else 0)
    for step in range(8):
        x = np.zeros((tokens, hidden), np.float32)
        for m in range(tokens):
            x[m, (417 + step + 97 * m) % hidden] = [8.0, -24.0, 40.0, 16.0, -8.0, 12.0, 20.0, 32.0][m]
        mlp.forward_mlp_prepared(dev_bf16(x, cuda), ws=ws)
        L.device_status()
        act_dev = host_f32(ws[tokens * (hidden + 2 * inter):tokens * (hidden + 3 * inter)].view(tokens, inter))
        _, _, act_cpu = o.ffn(layer, x, intermediates=True)
        ulp = np.maximum(np.abs(act_cpu), 2.0 ** -100) * 2.0 ** -7
        assert np.all(np.abs(act_dev - act_cpu) <= ulp)
        assert np.count_nonzero(act_dev != act_cpu) <= act_cpu.size // 50
    L.load().ffn_int4_set_decode_kernel(old)


@pytest.mark.parametrize("tokens", [1, 2, 8])
@pytest.mark.parametrize("poison", [float("nan"), float("inf")])
def test_non_finite_activation_gives_non_finite_output(cuda, tokens, poison):
    """The reference's FMA chain carries a NaN or an Inf in x into every row's sum
    (csrc/kernels/gemm_quant.cu:182-199).  Here a non-finite input element likewise makes every
    output of its token non-finite (all NaN where the reference would mix NaN and +-Inf); the other
    tokens of the call are untouched."""
    x, layers = o.draw_config(1024, 3072, 23, tokens=tokens)
    want = o.ffn(layers[0], x)
    mlp = upload_layer(layers[0], cuda)
    xd = dev_bf16(x, cuda).clone()
    xd[tokens - 1, 333] = poison
    y = host_f32(mlp.forward_mlp_prepared(xd))
    L.device_status()
    assert not np.isfinite(y[tokens - 1]).any()
    if tokens > 1:
        assert np.isfinite(y[:tokens - 1]).all()
        assert o.compare(y[:tokens - 1], want[:tokens - 1])[1] <= 5e-3
    g = ops.gemm_int4_bf16(xd, mlp.tensors[0], mlp.tensors[1])
    torch.cuda.synchronize()
    assert not np.isfinite(host_f32(g)[tokens - 1]).any()


def test_lm_head_and_projection_shaped_gemv(cuda):
    """The other weight-traffic-bound decode GEMVs of the model in this format (attention / GDN
    projections, the 248,320-row LM head; docs/plan-numeric-contract.md:1566-1569) through the
    streaming kernel, held to the reference's kernel gate (max_rel <= 8e-3, rms_rel <= 4e-3,
    tests/test_quantization_kernel.py:130-136).  Packed bytes and scales are drawn directly (every code
    in [-7, 7], scales around 2^-7), so no FP32 copy of the 1.27 G-element head is needed."""
    rng = np.random.default_rng(77)
    for n, k, m in [(248320, 5120, 1), (12288, 5120, 2), (5120, 6144, 1)]:
        lo = (rng.integers(0, 15, (n, k // 2), dtype=np.uint8).astype(np.int16) - 7) & 0xF
        hi = (rng.integers(0, 15, (n, k // 2), dtype=np.uint8).astype(np.int16) - 7) & 0xF
        packed = (lo | (hi << 4)).astype(np.uint8)
        del lo, hi
        scales = (0x3C00 + rng.integers(0, 128, (n, k // 128))).astype(np.uint16)
        x = o.bf16_round(rng.standard_normal((m, k), dtype=np.float32) * np.float32(0.5))
        ref = o.matmul_packed_f64(x, packed, scales)
        out = ops.gemm_int4_bf16(dev_bf16(x, cuda), dev_u8(packed, cuda), dev_bits(scales, cuda))
        L.device_status()
        err = np.abs(host_f32(out).astype(np.float64) - ref)
        scale = float(np.abs(ref).max())
        assert err.max() / scale <= 8e-3 and np.sqrt((err ** 2).mean()) / scale <= 4e-3, (n, k, m)
