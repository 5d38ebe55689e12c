"""Pins the CPU oracle (oracle/int4_format_oracle.c, oracle/ffn_oracle.py) against the reference's
own known-answer vectors for the INT4 format (tests/quantization_format_test.c), against the golden
fixtures generated from the reference's code (tests/golden/make_golden.py), and - where the
reference checkout was available to build oracle/_ref - bit-for-bit against the reference library.
"""
import ctypes
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import ffn_oracle as o

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_layout_refusals():
    # tests/quantization_format_test.c:48-75
    lib = o._lib()
    pb, sc = ctypes.c_longlong(), ctypes.c_longlong()
    ok = lambda n, k, g: lib.orc_layout(n, k, g, ctypes.byref(pb), ctypes.byref(sc))
    assert ok(8, 128, 128) == 0 and pb.value == 512 and sc.value == 8
    assert ok(8, 256, 128) == 0 and sc.value == 16
    assert ok(8, 192, 128) == 2     # 1.5 groups
    assert ok(12, 128, 128) == 2    # 1.5 tiles
    assert ok(0, 128, 128) == 2
    assert ok(8, -128, 128) == 2
    assert ok(8, 128, 64) == 2      # the group is part of the format
    assert lib.orc_layout(8, 128, 128, None, None) == 1


def test_bf16_vectors():
    # tests/quantization_format_test.c:81-103
    lib = o._lib()
    assert lib.orc_f32_to_bf16(1.0) == 0x3F80
    assert lib.orc_f32_to_bf16(-2.0) == 0xC000
    assert lib.orc_f32_to_bf16(0.0) == 0
    assert lib.orc_bf16_to_f32(0x3F80) == 1.0
    assert lib.orc_bf16_to_f32(0xC000) == -2.0
    assert lib.orc_f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80          # tie -> even
    assert lib.orc_f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82      # tie -> even (up)
    assert lib.orc_f32_to_bf16(3.4e38) in (0x7F80, 0x7F7F)
    v = np.array([1.0, -2.0, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8], np.float32)
    assert o.bf16_bits(v).tolist() == [0x3F80, 0xC000, 0x3F80, 0x3F82]


def test_hand_byte_pattern():
    # tests/quantization_format_test.c:118-174: codes {0,1,-1,-7,7,3,-3,2} with scale exactly 1.0
    w = np.zeros((8, 128), np.float32)
    w[0, :8] = [0, 1, -1, -7, 7, 3, -3, 2]
    packed, scales = o.quantize(w)
    assert o.bf16_to_f32(scales)[0, 0] == 1.0
    assert packed[0, :4].tolist() == [0x10, 0x9F, 0x37, 0x2D]
    lib = o._lib()
    codes = [lib.orc_packed_code(packed.ctypes.data, 0, k, 128) for k in range(8)]
    assert codes == [0, 1, -1, -7, 7, 3, -3, 2]
    back = o.dequantize(packed, scales)
    assert back[0, :8].tolist() == [0, 1, -1, -7, 7, 3, -3, 2]
    assert not back[0, 8:].any() and not back[1:].any()


def test_edge_groups():
    # tests/quantization_format_test.c:175-245
    w = np.zeros((8, 128), np.float32)
    packed, scales = o.quantize(w)
    assert (o.bf16_to_f32(scales) == 1.0).all() and not packed.any()       # zero group -> s = 1
    w[0, 0], w[0, 1] = 0.7000001, -0.7000001
    packed, scales = o.quantize(w)
    lib = o._lib()
    assert lib.orc_packed_code(packed.ctypes.data, 0, 0, 128) == 7
    assert lib.orc_packed_code(packed.ctypes.data, 0, 1, 128) == -7
    w[:] = 0
    w[0, 0] = 1e-40                                                          # scale rounds to zero
    with pytest.raises(ValueError):
        o.quantize(w)
    for bad in (np.nan, np.inf):
        w[:] = 0
        w[0, 5] = bad
        with pytest.raises(ValueError):
            o.quantize(w)
    w[:] = 0
    packed, scales = o.quantize(w)
    packed[0, 0] = 0x08                                                      # reserved code
    with pytest.raises(ValueError):
        o.dequantize(packed, scales)
    scales[0, 0] = 0                                                         # non-positive scale
    packed[0, 0] = 0
    with pytest.raises(ValueError):
        o.dequantize(packed, scales)


def test_requantize_is_fixed_point():
    rng = np.random.default_rng(5)
    w = rng.standard_normal((16, 512), dtype=np.float32) * np.float32(0.05)
    p, s = o.quantize(w)
    p2, s2 = o.quantize(o.dequantize(p, s))
    assert np.array_equal(p, p2) and np.array_equal(s, s2)


def test_reference_fixture():
    # the reference's deterministic [8, 256] fixture (tests/quantization_format_test.c:251-308),
    # emitted by the reference binary and committed as tests/golden/format_fixture.json
    with open(os.path.join(GOLDEN, "format_fixture.json")) as f:
        fx = json.load(f)
    n, k = fx["n"], fx["k"]
    w = np.array(fx["weights_f32_bits"], np.uint32).view(np.float32).reshape(n, k)
    # the fixture's definition, restated: w_i = ((i % 17) - 8) / 32 + (i % 3) / 128
    i = np.arange(n * k)
    assert np.array_equal(w.ravel(), ((i % 17) - 8).astype(np.float32) * np.float32(0.03125)
                          + (i % 3).astype(np.float32) * np.float32(0.0078125))
    packed, scales = o.quantize(w)
    assert packed.ravel().tolist() == fx["packed"]
    assert scales.ravel().tolist() == fx["scales_bf16"]
    deq = o.dequantize(packed, scales)
    assert deq.view(np.uint32).ravel().tolist() == fx["dequantized_f32_bits"]
    assert np.array_equal(o.dequantize_numpy(packed, scales).view(np.uint32), deq.view(np.uint32))


@pytest.mark.parametrize("cfg", [0, 1])
def test_config_digests(cfg):
    """The restatement reproduces the bytes the reference's quantizer made for the seeded configs."""
    with open(os.path.join(GOLDEN, "config_digests.json")) as f:
        want = json.load(f)[str(cfg)]
    x, layers = o.draw_config(want["hidden"], want["inter"], want["seed"])
    lay = layers[0]
    i = want["inter"]
    assert sha(o.bf16_bits(x)) == want["x_sha256"]
    assert sha(lay.gate_up_packed[:i]) == want["gate_packed_sha256"]
    assert sha(lay.gate_up_packed[i:]) == want["up_packed_sha256"]
    assert sha(lay.gate_up_scales[:i]) == want["gate_scales_sha256"]
    assert sha(lay.gate_up_scales[i:]) == want["up_scales_sha256"]
    assert sha(lay.down_packed) == want["down_packed_sha256"]
    assert sha(lay.down_scales) == want["down_scales_sha256"]
    if cfg == 0:
        assert sha(o.dequantize(lay.gate_up_packed[:i], lay.gate_up_scales[:i])) == want["gate_dequant_sha256"]
        assert sha(o.dequantize(lay.down_packed, lay.down_scales)) == want["down_dequant_sha256"]


def test_ffn_chain_golden():
    """Config 0's FFN output, computed when the fixture was made from weights the REFERENCE library
    quantized and dequantized, equals the oracle chain's output bit for bit."""
    with open(os.path.join(GOLDEN, "ffn_config0.json")) as f:
        fx = json.load(f)
    x, layers = o.draw_config(fx["hidden"], fx["inter"], fx["seed"])
    assert o.bf16_bits(x).ravel().tolist() == fx["x_bf16"]
    y, gu, act = o.ffn(layers[0], x, intermediates=True)
    assert sha(o.bf16_bits(act)) == fx["act_bf16_sha256"]
    assert o.bf16_bits(y).ravel().tolist() == fx["y_bf16"]


def test_against_reference_library():
    """Bit-for-bit against the reference's compiled linear_weight.cpp, when oracle/_ref exists."""
    ref = o.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref was not built (no reference checkout on this machine)")

    class Layout(ctypes.Structure):
        _fields_ = [(n, ctypes.c_longlong) for n in ("n", "k", "group", "packed_bytes", "scale_count")]

    rng = np.random.RandomState(11)
    for n, k in ((8, 128), (256, 128), (1024, 256), (64, 5120)):
        # the weight recipe of the reference's kernel gate, tests/test_quantization_kernel.py:100-104
        w = (rng.randn(n, k) * 0.05).astype(np.float32)
        w *= (1.0 + 0.5 * rng.rand(n, k // 128).astype(np.float32)).repeat(128, axis=1)
        w[0, :128] = 0.0
        lay = Layout()
        assert ref.linear_layout_init(ctypes.byref(lay), ctypes.c_longlong(n), ctypes.c_longlong(k),
                                      ctypes.c_longlong(128)) == 0
        p = np.zeros((n, k // 2), np.uint8)
        s = np.zeros((n, k // 128), np.uint16)
        assert ref.linear_quantize_int4(ctypes.byref(lay), ctypes.c_void_p(w.ctypes.data),
                                        ctypes.c_void_p(p.ctypes.data), ctypes.c_void_p(s.ctypes.data)) == 0
        d = np.empty((n, k), np.float32)
        assert ref.linear_dequantize_int4(ctypes.byref(lay), ctypes.c_void_p(p.ctypes.data),
                                          ctypes.c_void_p(s.ctypes.data), ctypes.c_void_p(d.ctypes.data)) == 0
        p2, s2 = o.quantize(w)
        assert np.array_equal(p, p2) and np.array_equal(s, s2)
        assert np.array_equal(o.dequantize(p2, s2).view(np.uint32), d.view(np.uint32))


def test_slice_rank_layout_and_refusal():
    """Per-rank slices keep the global scales; a split inside a group is refused by name
    (csrc/engine.cu:2316-2322; tests/test_quantized_sharding.py:99-119 uses intermediate=384)."""
    rng = np.random.default_rng(9)
    h, i = 256, 512
    lay = o.draw_layer(rng, h, i, False)
    full_gu = o.dequantize(lay.gate_up_packed, lay.gate_up_scales)
    full_d = o.dequantize(lay.down_packed, lay.down_scales)
    for tp in (1, 2, 4):
        for r in range(tp):
            gp, gs, dp, ds = o.slice_rank(lay.gate_up_packed, lay.gate_up_scales, lay.down_packed,
                                          lay.down_scales, tp, r)
            per = i // tp
            assert gp.shape == (2 * per, h // 2) and dp.shape == (h, per // 2)
            want = np.concatenate([full_gu[r * per:(r + 1) * per], full_gu[i + r * per:i + (r + 1) * per]])
            assert np.array_equal(o.dequantize(gp, gs), want)
            assert np.array_equal(o.dequantize(dp, ds), full_d[:, r * per:(r + 1) * per])
    lay384 = o.draw_layer(rng, 256, 384, False)
    with pytest.raises(ValueError, match="splits K at a non-group boundary"):
        o.slice_rank(lay384.gate_up_packed, lay384.gate_up_scales, lay384.down_packed,
                     lay384.down_scales, 2, 1)
    with pytest.raises(ValueError, match="does not divide"):
        o.slice_rank(lay.gate_up_packed, lay.gate_up_scales, lay.down_packed, lay.down_scales, 3, 0)
