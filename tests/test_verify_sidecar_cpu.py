"""ffn_verify_sidecar without a GPU (rederive_samples = 0): the checks and the wording of the reference
converter's --verify mode (scripts/quantize_weights.py:328-461) on a sidecar written in the
converter's layout, clean and then damaged in each way that mode is meant to catch."""
import ctypes
import hashlib
import json
import os

import pytest

from haskell_infer_demo_b200 import lib as L
from oracle import ffn_oracle as o
import sidecar_util

ROLES = ["embed", "postNorm", "mlpGate", "mlpUp", "mlpDown"]


def verify(root, samples=0):
    buf = ctypes.create_string_buffer(1 << 16)
    n = L.load().ffn_verify_sidecar(os.path.join(root, "weights.manifest.json").encode(), samples, buf, len(buf))
    return n, buf.value.decode()


@pytest.fixture()
def sidecar(tmp_path):
    """A two-layer sidecar with a real descriptor, a real source file and a full precision map."""
    root = str(tmp_path / "out")
    os.makedirs(root)
    _, layers = o.draw_config(256, 384, 21, layers=2)
    doc = sidecar_util.manifest_dict(root, layers)
    desc = {"num_layers": 2, "layer_ffns": ["dense", "dense"], "role_names": ROLES, "role_templates": ["t"] * len(ROLES)}
    desc_path = str(tmp_path / "desc.json")
    with open(desc_path, "w") as f:
        json.dump(desc, f)
    src_dir = str(tmp_path / "model")
    os.makedirs(src_dir)
    with open(os.path.join(src_dir, "model.safetensors"), "wb") as f:
        f.write(b"not read by the host checks" * 100)
    sha = lambda p: hashlib.sha256(open(p, "rb").read()).hexdigest()
    doc["descriptor"] = {"path": desc_path, "sha256": sha(desc_path)}
    doc["source"] = {"model_dir": src_dir, "files": [{"name": "model.safetensors", "bytes": 2700,
                                                      "sha256": sha(os.path.join(src_dir, "model.safetensors"))}]}
    doc["precision_map"] = [{"checkpoint_tensor": "t", "layer": l, "role": r,
                             "precision": "int4" if r.startswith("mlp") else "bf16"} for l in range(2) for r in ROLES]

    def write(d=doc):
        with open(os.path.join(root, "weights.manifest.json"), "w") as f:
            f.write(sidecar_util.dumps(d))
    write()
    return root, doc, write, src_dir, desc_path


def test_clean_sidecar_verifies(sidecar):
    root, doc, _, _, _ = sidecar
    n, report = verify(root)
    assert n == 0, report
    assert report == ("verify: 6 entries, 2 pair(s) match their members' rows, the precision map covers 10 (role, layer) "
                      "cells, the source is unchanged\n")


def test_damaged_artifacts_are_named(sidecar):
    root, doc, _, _, _ = sidecar
    path = os.path.join(root, "artifacts", "mlpGate_layer0.packed")
    raw = bytearray(open(path, "rb").read())
    raw[7] ^= 0x10
    open(path, "wb").write(bytes(raw))
    n, report = verify(root)
    assert n == 2
    assert "verify: (0, 'mlpGate') payload does not match its checksum\n" in report
    assert "verify: pair at layer 0 is not its members' packed rows in order\n" in report

    scales = os.path.join(root, "artifacts", "mlpDown_layer1.scales")
    size = os.path.getsize(scales)
    kept = open(scales, "rb").read()[:-2]
    open(scales, "wb").write(kept)
    n, report = verify(root)
    assert f"verify: (1, 'mlpDown') scales are {size - 2} bytes, expected {size}\n" in report
    assert "verify: (1, 'mlpDown') scales do not match their checksum\n" in report

    os.remove(os.path.join(root, "artifacts", "mlpUp_layer1.packed"))
    n, report = verify(root)
    assert "verify: (1, 'mlpUp') has no payload at artifacts/mlpUp_layer1.packed\n" in report
    assert "verify: pair at layer 1 is missing an artifact\n" in report


def test_manifest_claims_are_rederived(sidecar):
    root, doc, write, src_dir, desc_path = sidecar
    bad = json.loads(json.dumps(doc))
    bad["format"]["arithmetic"] = "something else"
    bad["format"]["group"] = 64
    bad["entries"].append(bad["entries"][0])
    bad["precision_map"] = [c for c in bad["precision_map"] if not (c["layer"] == 1 and c["role"] == "embed")]
    bad["precision_map"][0]["precision"] = "int4"                      # (0, 'embed') has no entry
    bad["pairs"][0]["logical_shape"] = [1, 2]
    bad["pairs"][1]["members"][1]["role"] = "mlpSideways"
    write(bad)
    n, report = verify(root)
    for line in ("verify: the format's arithmetic is something else, expected csrc/linear_weight.cpp (the Q0 reference)\n",
                 "verify: the format's group is 64, expected 128\n",
                 "verify: (0, 'mlpGate') appears twice\n",
                 "verify: the precision map and the entries disagree about (0, 'embed')\n",
                 "verify: the precision map does not cover layer 1's embed\n",
                 "verify: pair at layer 0 claims another shape than [768, 256]\n",
                 "verify: pair at layer 1 names a member that has no entry\n"):
        assert line in report, (line, report)
    assert n == report.count("\n")


def test_source_and_descriptor_are_checked(sidecar):
    root, doc, write, src_dir, desc_path = sidecar
    with open(os.path.join(src_dir, "model.safetensors"), "ab") as f:
        f.write(b"!")
    with open(desc_path, "a") as f:
        f.write(" ")
    n, report = verify(root)
    assert "verify: the source file model.safetensors no longer matches its checksum\n" in report
    assert "verify: the descriptor no longer matches its checksum\n" in report
    os.remove(os.path.join(src_dir, "model.safetensors"))
    n, report = verify(root)
    assert "verify: the source file model.safetensors is gone\n" in report


def test_unreadable_manifest_is_a_status_not_a_count(tmp_path):
    assert verify(str(tmp_path))[0] == -3
    (tmp_path / "weights.manifest.json").write_text("[1, 2]")
    assert verify(str(tmp_path))[0] == -3


def test_rederiving_needs_the_gpu(sidecar):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this machine has a GPU")
    root, _, _, _, _ = sidecar
    n, _ = verify(root, samples=2)
    assert n < 0 and L.load().ffn_int4_last_error()       # the source here is not a checkpoint, and there is no GPU: no silent pass
