"""ffn_convert_checkpoint end to end on a GPU: a synthetic BF16 safetensors checkpoint is converted; the
artifacts must be byte-identical to what the reference's quantizer arithmetic (the CPU oracle) makes
of the same tensors, the manifest must be the document the reference's converter would write
(scripts/quantize_weights.py:219-320) apart from the converter's name, both strict readers must accept
it, and the loader must be able to run an FFN from it."""
import ctypes
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200.lib import MlpWeights
from oracle import ffn_oracle as o
from gpu_util import assert_ffn_close, dev_bf16, host_f32
from test_converter_cpu import convert, descriptor, model

pytestmark = pytest.mark.gpu

ROLES = {"mlpGate": "gate", "mlpUp": "up", "mlpDown": "down"}


def sha(raw):
    return hashlib.sha256(raw).hexdigest()


def artifact(root, rel):
    with open(os.path.join(root, rel), "rb") as f:
        return f.read()


def test_conversion_end_to_end(cuda, tmp_path):
    layers, hidden, inter = 2, 256, 512
    d, desc, tensors = model(tmp_path, layers=layers, hidden=hidden, inter=inter)
    out = str(tmp_path / "out")
    st, msg = convert(d, desc, out)
    assert st == 0, msg
    with open(os.path.join(out, "weights.manifest.json")) as f:
        text = f.read()
    doc = json.loads(text)
    assert text == json.dumps(doc, indent=2, sort_keys=True) + "\n"          # the reference converter's encoding

    # artifacts: the bytes the reference's arithmetic makes of the same (BF16-valued) tensors
    quantized, err_max, err_sq, elems = {}, 0.0, 0.0, 0
    for l in range(layers):
        for role, short in ROLES.items():
            src = tensors[f"model.layers.{l}.mlp.{short}_proj.weight"]
            p, s = o.quantize(src)
            quantized[(l, role)] = (p, s)
            assert artifact(out, f"artifacts/{role}_layer{l}.packed") == p.tobytes()
            assert artifact(out, f"artifacts/{role}_layer{l}.scales") == s.tobytes()
            diff = np.abs(src - o.dequantize(p, s))
            err_max = max(err_max, float(diff.max()))
            err_sq += float((diff.astype(np.float64) ** 2).sum())
            elems += diff.size
        gp = quantized[(l, "mlpGate")][0].tobytes() + quantized[(l, "mlpUp")][0].tobytes()
        gs = quantized[(l, "mlpGate")][1].tobytes() + quantized[(l, "mlpUp")][1].tobytes()
        assert artifact(out, f"artifacts/mlpGateUp_layer{l}.packed") == gp
        assert artifact(out, f"artifacts/mlpGateUp_layer{l}.scales") == gs

    # the manifest, field by field, as scripts/quantize_weights.py builds it
    names = descriptor(layers)["role_names"]
    assert doc["manifest_version"] == 1 and doc["converter"]["version"] == 1 and doc["converter"]["name"]
    assert (doc["format"]["group"], doc["format"]["qmin"], doc["format"]["qmax"], doc["format"]["invalid_code"],
            doc["format"]["zero_point"], doc["format"]["packed_dtype"], doc["format"]["scale_dtype"],
            doc["format"]["abi_version"], doc["format"]["name"]) == (128, -7, 7, -8, 0, "u8", "bf16", 1,
                                                                     "int4_symmetric_group_bf16_scale")
    assert len(doc["entries"]) == 3 * layers and len(doc["pairs"]) == layers
    at = 0
    for l in range(layers):
        for role, short in ROLES.items():
            e = doc["entries"][at]
            at += 1
            p, s = quantized[(l, role)]
            n, k = p.shape[0], p.shape[1] * 2
            assert e == {
                "role": role, "role_index": names.index(role), "layer": l,
                "checkpoint_tensor": f"model.layers.{l}.mlp.{short}_proj.weight",
                "logical_shape": [n, k], "local_shape": [n, k], "group_axis": "k", "group": 128,
                "packed": {"file": f"artifacts/{role}_layer{l}.packed", "dtype": "u8", "bytes": p.size, "sha256": sha(p.tobytes())},
                "scales": {"file": f"artifacts/{role}_layer{l}.scales", "dtype": "bf16", "count": s.size, "bytes": s.size * 2,
                           "sha256": sha(s.tobytes())},
            }
        pair = doc["pairs"][l]
        assert pair["name"] == "mlpGateUp" and pair["layer"] == l and pair["group"] == 128
        assert pair["members"] == [{"role": "mlpGate", "role_index": names.index("mlpGate")},
                                   {"role": "mlpUp", "role_index": names.index("mlpUp")}]
        assert pair["logical_shape"] == [2 * inter, hidden] and pair["rule"].startswith("row concatenation: gate rows then up rows")
        assert pair["packed"]["sha256"] == sha(artifact(out, pair["packed"]["file"])) and pair["packed"]["bytes"] == inter * hidden
        assert pair["scales"]["sha256"] == sha(artifact(out, pair["scales"]["file"])) and pair["scales"]["count"] == 2 * inter * hidden // 128
    assert len(doc["precision_map"]) == layers * len(names)
    for cell in doc["precision_map"]:
        assert cell["precision"] == ("int4" if cell["role"] in ROLES else "bf16")
    src_file = os.path.join(str(d), "model-00001-of-00001.safetensors")
    assert doc["source"]["files"] == [{"name": "model-00001-of-00001.safetensors", "bytes": os.path.getsize(src_file),
                                       "sha256": sha(open(src_file, "rb").read())}]
    assert doc["descriptor"]["sha256"] == sha(open(str(desc), "rb").read())
    qe = doc["quantization_error"]
    assert qe["elements"] == elems and qe["max_abs"] == err_max
    assert qe["rms"] == pytest.approx((err_sq / elems) ** 0.5, rel=1e-9)

    # both strict readers accept the document
    lib = L.load()
    handle = ctypes.c_void_p()
    assert lib.ffn_quant_manifest_parse(text.encode(), ctypes.byref(handle)) == 0, lib.ffn_int4_last_error()
    lib.ffn_quant_manifest_free(handle)
    ref = o.ref_lib("libref_quant_manifest.so")
    if ref is not None:
        buf = ctypes.create_string_buffer(2 << 20)
        ref.quant_manifest_parse.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
        assert ref.quant_manifest_parse(text.encode(), buf, None, 0) == 0

    # and the loader runs an FFN from it
    loaded = ctypes.c_void_p()
    assert lib.ffn_load_quantized_ffn(out.encode(), layers, hidden, inter, 1, 0, ctypes.byref(loaded)) == 0, lib.ffn_int4_last_error()
    x = o.bf16_round(np.random.default_rng(9).standard_normal((1, hidden), dtype=np.float32))
    for l in range(layers):
        w = MlpWeights()
        assert lib.ffn_quantized_ffn_layer(loaded, l, ctypes.byref(w)) == 0
        dims = L.ModelDims()
        dims.hidden_size, dims.intermediate_size, dims.max_chunk = hidden, inter, 128
        xd = dev_bf16(x, cuda)
        ws = torch.empty(hidden + 3 * inter, dtype=torch.bfloat16, device=cuda)
        y = torch.empty((1, hidden), dtype=torch.bfloat16, device=cuda)
        L.check(lib.ffn_forward_mlp_prepared(None, None, ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(ws.data_ptr()),
                                             ctypes.c_void_p(y.data_ptr()), ctypes.byref(w), 1, ctypes.byref(dims)))
        L.device_status()
        lay = o.Layer(np.concatenate([quantized[(l, "mlpGate")][0], quantized[(l, "mlpUp")][0]]),
                      np.concatenate([quantized[(l, "mlpGate")][1], quantized[(l, "mlpUp")][1]]),
                      quantized[(l, "mlpDown")][0], quantized[(l, "mlpDown")][1], None)
        assert_ffn_close(host_f32(y), o.ffn(lay, x), f"layer {l} from the converted checkpoint")
    assert lib.ffn_quantized_ffn_free(loaded) == 0


def test_limit_layers_and_moe_layers_are_left_in_bf16(cuda, tmp_path):
    d, desc, _ = model(tmp_path, layers=2)
    doc_desc = descriptor(2, ffns=["dense", "moe"])
    (tmp_path / "mixed.json").write_text(json.dumps(doc_desc))
    out = str(tmp_path / "mixed")
    st, msg = convert(d, tmp_path / "mixed.json", out)
    assert st == 0, msg
    doc = json.load(open(os.path.join(out, "weights.manifest.json")))
    assert [e["layer"] for e in doc["entries"]] == [0, 0, 0] and len(doc["pairs"]) == 1
    assert all(c["precision"] == "bf16" for c in doc["precision_map"] if c["layer"] == 1)
    out1 = str(tmp_path / "first")
    st, msg = convert(d, desc, out1, limit=1)
    assert st == 0, msg
    assert [e["layer"] for e in json.load(open(os.path.join(out1, "weights.manifest.json")))["entries"]] == [0, 0, 0]


def test_unrepresentable_group_is_refused_with_the_quantizers_message(cuda, tmp_path):
    d, desc, tensors = model(tmp_path)
    bad = dict(tensors)
    w = tensors["model.layers.0.mlp.up_proj.weight"].copy()
    w[5, 128:256] = np.float32(1e-40)
    bad["model.layers.0.mlp.up_proj.weight"] = w
    bd = tmp_path / "bad"
    bd.mkdir()
    from test_converter_cpu import write_safetensors
    write_safetensors(str(bd / "m.safetensors"), bad)
    st, msg = convert(bd, desc, tmp_path / "out")
    assert st == -3 and "row 5 group 1" in msg
    assert not os.path.exists(tmp_path / "out" / "weights.manifest.json")


def test_verify_rederives_from_the_source(cuda, tmp_path):
    """The converter's output passes ffn_verify_sidecar including the re-derivation of sampled entries
    from the source checkpoint; an artifact altered together with its recorded digest passes every
    host check and is caught only by that re-derivation."""
    from test_verify_sidecar_cpu import verify
    d, desc, _ = model(tmp_path, layers=1)
    out = str(tmp_path / "out")
    st, msg = convert(d, desc, out)
    assert st == 0, msg
    n, report = verify(out, samples=2)
    assert n == 0, report
    assert report.endswith("the source is unchanged and the sampled artifacts re-derive from it\n")

    path = os.path.join(out, "artifacts", "mlpGate_layer0.packed")
    raw = bytearray(open(path, "rb").read())
    raw[3] ^= 0x01
    open(path, "wb").write(bytes(raw))
    manifest_path = os.path.join(out, "weights.manifest.json")
    doc = json.load(open(manifest_path))
    doc["entries"][0]["packed"]["sha256"] = sha(bytes(raw))
    assert doc["entries"][0]["role"] == "mlpGate"
    with open(manifest_path, "w") as f:
        f.write(json.dumps(doc, indent=2, sort_keys=True) + "\n")
    n, report = verify(out, samples=2)
    assert "verify: mlpGate_0 does not re-derive from the source\n" in report
    assert "verify: pair at layer 0 is not its members' packed rows in order\n" in report
    assert n == 2, report
