"""Host side of the converter (ffn_convert_checkpoint), without a GPU: its JSON encoder against
Python's json.dumps(indent=2, sort_keys=True), which is how the reference's converter writes the
manifest (scripts/quantize_weights.py:318-320), and the refusals that come before any tensor reaches
the GPU, on a synthetic BF16 safetensors checkpoint."""
import ctypes
import json
import os
import struct

import numpy as np
import pytest

from haskell_infer_demo_b200 import lib as L
from oracle import ffn_oracle as o


def reencode(doc):
    text = json.dumps(doc)
    buf = ctypes.create_string_buffer(len(text) * 8 + 4096)
    st = L.load().ffn_json_reencode(text.encode(), buf, len(buf))
    assert st == 0, L.load().ffn_int4_last_error()
    return buf.value.decode()


def test_encoder_matches_python():
    rng = np.random.default_rng(7)
    floats = [0.0, 1.0, -1.5, 0.1, 1e-5, 1.5e-5, 0.0001, 0.00012345, 123456789.125, 1e15, 1e16, 1.2345e16, 1e22, 5e-324,
              1.7976931348623157e308, 2.0 ** -20, 2.0 ** -24, 2.0 ** -1074, 2.0 ** 70, 1 / 3, 0.004241943359375, float(np.float32(0.0032958984)),
              float(np.float32(1.1920929e-07))]
    floats += [float(x) for x in rng.standard_normal(200) * 10.0 ** rng.integers(-12, 12, 200)]
    floats += [float(np.float32(x)) for x in rng.standard_normal(100) * 1e-3]
    doc = {
        "zeta": floats, "alpha": {"b": [], "a": {}, "c": [1, -2, 3000000000000]}, "mid": "plain",
        "text": "quote \" backslash \\ tab \t newline \n bell \x07 del \x7f", "unicode": "Grüße, 世界, 🙂",
        "nested": [[1, [2, [3]]], {"k": [{"deep": 1.25}]}], "path": "/tmp/model dir/x.json", "Upper": 1, "_under": 2,
    }
    assert reencode(doc) == json.dumps(doc, indent=2, sort_keys=True)
    for small in ({}, [], {"a": []}, [[]], {"only": 1}):
        assert reencode(small) == json.dumps(small, indent=2, sort_keys=True)


def write_safetensors(path, tensors, dtype="BF16"):
    """tensors: name -> float32 array holding BF16 values (or any array when dtype is not BF16)."""
    header, blobs, at = {}, [], 0
    for name, arr in tensors.items():
        raw = o.bf16_bits(arr).tobytes() if dtype == "BF16" else np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    header["__metadata__"] = {"format": "pt"}
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def descriptor(layers, ffns=None):
    return {
        "num_layers": layers, "layer_ffns": ffns or ["dense"] * layers,
        "role_names": ["embed", "postNorm", "mlpGate", "mlpUp", "mlpDown"],
        "role_templates": ["model.embed_tokens.weight", "model.layers.%d.post_attention_layernorm.weight",
                           "model.layers.%d.mlp.gate_proj.weight", "model.layers.%d.mlp.up_proj.weight",
                           "model.layers.%d.mlp.down_proj.weight"],
        "hidden_size": 256, "intermediate_size": 512,
    }


def model(tmp_path, layers=1, hidden=256, inter=512, seed=3):
    rng = np.random.default_rng(seed)
    tensors = {"model.embed_tokens.weight": o.bf16_round(rng.standard_normal((16, hidden), dtype=np.float32))}
    for l in range(layers):
        tensors[f"model.layers.{l}.mlp.gate_proj.weight"] = o.bf16_round(rng.standard_normal((inter, hidden), dtype=np.float32) * np.float32(0.02))
        tensors[f"model.layers.{l}.mlp.up_proj.weight"] = o.bf16_round(rng.standard_normal((inter, hidden), dtype=np.float32) * np.float32(0.02))
        tensors[f"model.layers.{l}.mlp.down_proj.weight"] = o.bf16_round(rng.standard_normal((hidden, inter), dtype=np.float32) * np.float32(0.02))
    d = tmp_path / "model"
    d.mkdir()
    write_safetensors(str(d / "model-00001-of-00001.safetensors"), tensors)
    desc = tmp_path / "desc.json"
    desc.write_text(json.dumps(descriptor(layers)))
    return d, desc, tensors


def convert(model_dir, desc, out, limit=-1):
    lib = L.load()
    st = lib.ffn_convert_checkpoint(str(model_dir).encode(), str(desc).encode(), str(out).encode(), None, 0, limit)
    return st, lib.ffn_int4_last_error().decode()


def test_refusals_before_the_gpu(tmp_path):
    d, desc, tensors = model(tmp_path)
    out = tmp_path / "out"
    # a descriptor whose role names and templates differ
    bad = descriptor(1)
    bad["role_templates"] = bad["role_templates"][:-1]
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    st, msg = convert(d, tmp_path / "bad.json", out)
    assert st == -4 and "role names and templates differ" in msg
    st, msg = convert(d, tmp_path / "missing.json", out)
    assert st == -4 and "cannot read" in msg
    # a tensor the descriptor names is not in the checkpoint
    (tmp_path / "two.json").write_text(json.dumps(descriptor(2)))
    st, msg = convert(d, tmp_path / "two.json", out, limit=-1)
    assert st != 0
    # ... which limit_layers = 1 never reaches; on a machine without a GPU the first tensor then fails loudly
    # a source that is not BF16
    f32 = tmp_path / "f32"
    f32.mkdir()
    write_safetensors(str(f32 / "m.safetensors"), tensors, dtype="F32")
    st, msg = convert(f32, desc, out)
    assert st == -3 and "only BF16 sources are admitted, got F32" in msg
    # the same tensor in two shards
    dup = tmp_path / "dup"
    dup.mkdir()
    write_safetensors(str(dup / "a.safetensors"), tensors)
    write_safetensors(str(dup / "b.safetensors"), {"model.embed_tokens.weight": tensors["model.embed_tokens.weight"]})
    st, msg = convert(dup, desc, out)
    assert st == -3 and "appears in two shards" in msg
    # a weight that is not 2-D
    flat = dict(tensors)
    flat["model.layers.0.mlp.gate_proj.weight"] = tensors["model.layers.0.mlp.gate_proj.weight"].reshape(-1)
    fd = tmp_path / "flat"
    fd.mkdir()
    write_safetensors(str(fd / "m.safetensors"), flat)
    st, msg = convert(fd, desc, out)
    assert st == -3 and "is not a 2-D weight" in msg


def test_no_cpu_fallback(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this machine has a GPU")
    d, desc, _ = model(tmp_path)
    st, msg = convert(d, desc, tmp_path / "out")
    assert st < 0 and msg
    assert not os.path.exists(tmp_path / "out" / "weights.manifest.json")


def test_encoder_matches_python_on_random_documents():
    """Property check (hypothesis): any document of integers, finite floats, text, lists and dictionaries."""
    from hypothesis import given, settings, strategies as st

    # text from the basic plane (keys beyond it sort by UTF-16 units in Python and by bytes here; manifests
    # have ASCII keys, and a value beyond the basic plane is in the fixed document above)
    text = st.text(alphabet=st.characters(max_codepoint=0xFFFF, exclude_categories=["Cs"]), max_size=12)
    leaves = st.one_of(st.integers(min_value=-(10 ** 15), max_value=10 ** 15),
                       st.floats(allow_nan=False, allow_infinity=False), text)
    docs = st.recursive(leaves, lambda kids: st.one_of(st.lists(kids, max_size=4),
                                                       st.dictionaries(text.filter(len), kids, max_size=4)),
                        max_leaves=25)

    @settings(max_examples=300, deadline=None)
    @given(docs)
    def check(doc):
        if not isinstance(doc, (list, dict)):
            doc = [doc]
        assert reencode(doc) == json.dumps(doc, indent=2, sort_keys=True)

    check()
