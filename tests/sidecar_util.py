"""Writes a quantized sidecar (weights.manifest.json + artifacts/) for synthetic layers, in the layout
the reference's converter produces (scripts/quantize_weights.py:42-56, 219-234, 260-276, 295-318):
sorted keys, two-space indent, raw little-endian artifacts without headers, a gate||up pair per layer.
Test data only."""
import hashlib
import json
import os

import numpy as np

ROLE_INDEX = {"mlpGate": 3, "mlpUp": 4, "mlpDown": 5}
FORMAT = {
    "abi_version": 1, "arithmetic": "csrc/linear_weight.cpp (the Q0 reference)", "group": 128, "invalid_code": -8,
    "name": "int4_symmetric_group_bf16_scale", "packed_dtype": "u8",
    "packing": "two_twos_complement_nibbles_per_byte_lower_k_index_in_low_nibble", "qmax": 7, "qmin": -7,
    "scale_dtype": "bf16", "zero_point": 0,
}


def _artifact(root, name, data, dtype, count=None):
    path = os.path.join("artifacts", name)
    raw = np.ascontiguousarray(data).tobytes()
    with open(os.path.join(root, path), "wb") as f:
        f.write(raw)
    rec = {"bytes": len(raw), "dtype": dtype, "file": path, "sha256": hashlib.sha256(raw).hexdigest()}
    if count is not None:
        rec["count"] = count
    return rec


def manifest_dict(root, layers):
    """layers: list of oracle Layer objects (gate_up pair [2I, H], down [H, I])."""
    os.makedirs(os.path.join(root, "artifacts"), exist_ok=True)
    entries, pairs, cells = [], [], []
    for l, lay in enumerate(layers):
        i, h = lay.inter, lay.hidden
        parts = {"mlpGate": (lay.gate_up_packed[:i], lay.gate_up_scales[:i], i, h),
                 "mlpUp": (lay.gate_up_packed[i:], lay.gate_up_scales[i:], i, h),
                 "mlpDown": (lay.down_packed, lay.down_scales, h, i)}
        for role, (p, s, n, k) in parts.items():
            tensor = f"model.layers.{l}.mlp.{ {'mlpGate': 'gate', 'mlpUp': 'up', 'mlpDown': 'down'}[role]}_proj.weight"
            entries.append({
                "checkpoint_tensor": tensor, "group": 128, "group_axis": "k", "layer": l,
                "local_shape": [n, k], "logical_shape": [n, k],
                "packed": _artifact(root, f"{role}_layer{l}.packed", p, "u8"),
                "role": role, "role_index": ROLE_INDEX[role],
                "scales": _artifact(root, f"{role}_layer{l}.scales", s, "bf16", count=int(s.size)),
            })
            cells.append({"checkpoint_tensor": tensor, "layer": l, "precision": "int4", "role": role})
        pairs.append({
            "group": 128, "layer": l, "logical_shape": [2 * i, h],
            "members": [{"role": "mlpGate", "role_index": 3}, {"role": "mlpUp", "role_index": 4}],
            "name": "mlpGateUp",
            "packed": _artifact(root, f"mlpGateUp_layer{l}.packed", lay.gate_up_packed, "u8"),
            "rule": "row concatenation: gate rows then up rows",
            "scales": _artifact(root, f"mlpGateUp_layer{l}.scales", lay.gate_up_scales, "bf16",
                                count=int(lay.gate_up_scales.size)),
        })
    cells.append({"checkpoint_tensor": "model.embed_tokens.weight", "layer": 0, "precision": "bf16", "role": "embed"})
    return {
        "converter": {"name": "scripts/quantize_weights.py", "version": 1},
        "descriptor": {"path": "synthetic", "sha256": "1" * 64},
        "entries": entries, "format": dict(FORMAT), "manifest_version": 1, "pairs": pairs,
        "precision_map": cells,
        "quantization_error": {"max_abs": 0.0, "note": "synthetic", "rms": 0.0},
        "source": {"files": [], "model_dir": "synthetic"},
    }


def dumps(doc):
    return json.dumps(doc, indent=2, sort_keys=True) + "\n"


def write_sidecar(root, layers):
    doc = manifest_dict(root, layers)
    with open(os.path.join(root, "weights.manifest.json"), "w") as f:
        f.write(dumps(doc))
    return doc
