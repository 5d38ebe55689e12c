"""Generates the committed golden fixtures from the REFERENCE's own code.

Run in a container that has the reference checkout (oracle/Makefile builds oracle/_ref from it):

    make -C oracle && python tests/golden/make_golden.py

Writes, next to this script:
  format_fixture.json   the reference's deterministic [8, 256] fixture, exactly as
                        `test_quantization_format --emit` prints it (weights, packed bytes, scales
                        and dequantized bits; tests/quantization_format_test.c:251-308)
  config_digests.json   SHA-256 of the packed payload and the scales of every synthetic
                        configuration's first layer, quantized by the reference's
                        linear_quantize_int4 (csrc/linear_weight.cpp:108-176), plus SHA-256 of the
                        reference's dequantization of config 0 - so a box without the reference can
                        still prove its restatement produces the reference's bytes
  ffn_config0.json      the oracle chain's output bits for config 0 with the weights quantized and
                        dequantized by the reference library
"""
import ctypes
import hashlib
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import ffn_oracle as o  # noqa: E402


class Layout(ctypes.Structure):
    _fields_ = [(n, ctypes.c_longlong) for n in ("n", "k", "group", "packed_bytes", "scale_count")]


def ref_quantize(ref, w):
    n, k = w.shape
    lay = Layout()
    assert ref.linear_layout_init(ctypes.byref(lay), ctypes.c_longlong(n), ctypes.c_longlong(k),
                                  ctypes.c_longlong(128)) == 0
    packed = np.zeros((n, k // 2), np.uint8)
    scales = np.zeros((n, k // 128), np.uint16)
    st = ref.linear_quantize_int4(ctypes.byref(lay), ctypes.c_void_p(w.ctypes.data),
                                  ctypes.c_void_p(packed.ctypes.data), ctypes.c_void_p(scales.ctypes.data))
    assert st == 0
    return packed, scales, lay


def ref_dequantize(ref, packed, scales, lay):
    out = np.empty((lay.n, lay.k), np.float32)
    st = ref.linear_dequantize_int4(ctypes.byref(lay), ctypes.c_void_p(packed.ctypes.data),
                                    ctypes.c_void_p(scales.ctypes.data), ctypes.c_void_p(out.ctypes.data))
    assert st == 0
    return out


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    ref = o.ref_lib()
    binary = os.path.join(ROOT, "oracle", "_ref", "test_quantization_format")
    if ref is None or not os.path.exists(binary):
        raise SystemExit("oracle/_ref is missing: run `make -C oracle` where the reference checkout exists")
    subprocess.run([binary, "--emit", os.path.join(HERE, "format_fixture.json")], check=True)

    digests = {}
    for cfg, spec in o.CONFIGS.items():
        rng = np.random.default_rng(spec["seed"])
        h, i = spec["hidden"], spec["inter"]
        x = o.bf16_round(rng.standard_normal((1, h), dtype=np.float32))
        entry = {"hidden": h, "inter": i, "seed": spec["seed"], "x_sha256": sha(o.bf16_bits(x))}
        tensors = {}
        for name, shape in (("gate", (i, h)), ("up", (i, h)), ("down", (h, i))):
            w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
            p, s, lay = ref_quantize(ref, w)
            entry[name + "_packed_sha256"] = sha(p)
            entry[name + "_scales_sha256"] = sha(s)
            tensors[name] = (p, s, lay)
            if cfg == 0:
                entry[name + "_dequant_sha256"] = sha(ref_dequantize(ref, p, s, lay))
        digests[str(cfg)] = entry
        if cfg == 0:
            layer = o.Layer(np.concatenate([tensors["gate"][0], tensors["up"][0]]),
                            np.concatenate([tensors["gate"][1], tensors["up"][1]]),
                            tensors["down"][0], tensors["down"][1])
            w_gu = np.concatenate([ref_dequantize(ref, *tensors["gate"]), ref_dequantize(ref, *tensors["up"])])
            w_d = ref_dequantize(ref, *tensors["down"])
            gu = o.bf16_round(o.matmul_f64(x, w_gu).astype(np.float32))
            act = o.silu_mul(gu[:, :i], gu[:, i:])
            y = o.bf16_round(o.matmul_f64(act, w_d).astype(np.float32))
            assert np.array_equal(o.bf16_bits(y), o.bf16_bits(o.ffn(layer, x)))
            with open(os.path.join(HERE, "ffn_config0.json"), "w") as f:
                json.dump({"hidden": h, "inter": i, "seed": 0,
                           "x_bf16": o.bf16_bits(x).ravel().tolist(),
                           "act_bf16_sha256": sha(o.bf16_bits(act)),
                           "y_bf16": o.bf16_bits(y).ravel().tolist()}, f)
        print("config", cfg, "done", flush=True)
    with open(os.path.join(HERE, "config_digests.json"), "w") as f:
        json.dump(digests, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
