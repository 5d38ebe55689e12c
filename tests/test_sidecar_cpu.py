"""CPU checks of the artifact path in libffn_int4.so (SHA-256, manifest reader, artifact read, shard
view) against the reference's known answers (tests/manifest_test.c:196-205 SHA vectors;
tests/quant_manifest_test.c:296-360 refusals, 364-435 artifact read; tests/model_desc_test.c:293-333
shard views) and, where oracle/_ref holds the reference's compiled quant_manifest.c, status for status
against the reference reader on the same documents."""
import ctypes
import hashlib
import os

import numpy as np
import pytest

from haskell_infer_demo_b200 import lib as L
from oracle import ffn_oracle as o
import sidecar_util

OK, ARG, SYNTAX, FORMAT, SHAPE, IO, HASH = range(7)


def parse(text):
    lib = L.load()
    h = ctypes.c_void_p()
    st = lib.ffn_quant_manifest_parse(text.encode(), ctypes.byref(h))
    return st, h


def ref_parse_status(text):
    ref = o.ref_lib("libref_quant_manifest.so")
    if ref is None:
        return None
    buf = ctypes.create_string_buffer(2 << 20)      # struct QuantManifest is ~1 MiB
    ref.quant_manifest_parse.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return ref.quant_manifest_parse(text.encode(), buf, None, 0)


@pytest.fixture(scope="module")
def fixture_text(tmp_path_factory):
    """Same shape as the reference's hand-written fixture: gate [256,256], up [128,256] ... our writer
    emits equal gate/up rows, so gate and up are both [256,256] and the pair [512,256]."""
    root = tmp_path_factory.mktemp("sidecar")
    rng = np.random.default_rng(3)
    lay = o.draw_layer(rng, 256, 256, False)
    doc = sidecar_util.manifest_dict(str(root), [lay])
    doc["entries"] = [e for e in doc["entries"] if e["role"] != "mlpDown"]
    doc["precision_map"] = [c for c in doc["precision_map"] if c["role"] != "mlpDown"]
    return sidecar_util.dumps(doc)


def test_sha256_known_answers():
    lib = L.load()
    out = ctypes.create_string_buffer(65)
    for msg in (b"", b"abc", b"abcdbcdecdefdefgefghfghighijhijkijkljklmklmnlmnomnopnopq", b"a" * 1000000,
                bytes(range(256)) * 37):
        assert lib.ffn_sha256_hex(msg, len(msg), out) == 0
        assert out.value.decode() == hashlib.sha256(msg).hexdigest()
    lib.ffn_sha256_hex(b"abc", 3, out)
    assert out.value == b"ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"


def test_fixture_parses_and_lookups(fixture_text):
    lib = L.load()
    st, h = parse(fixture_text)
    assert st == OK, lib.ffn_int4_last_error()
    assert ref_parse_status(fixture_text) in (None, OK)
    e, p, i4, b16 = (ctypes.c_int() for _ in range(4))
    lib.ffn_quant_manifest_counts(h, ctypes.byref(e), ctypes.byref(p), ctypes.byref(i4), ctypes.byref(b16))
    assert (e.value, p.value, i4.value, b16.value) == (2, 1, 2, 1)
    gate = lib.ffn_quant_manifest_find_entry(h, 0, b"mlpGate")
    assert gate >= 0 and lib.ffn_quant_manifest_find_entry(h, 1, b"mlpGate") < 0
    n, k, g, ri = ctypes.c_longlong(), ctypes.c_longlong(), ctypes.c_longlong(), ctypes.c_int()
    lib.ffn_quant_manifest_entry_shape(h, gate, ctypes.byref(n), ctypes.byref(k), ctypes.byref(g), ctypes.byref(ri))
    assert (n.value, k.value, g.value, ri.value) == (256, 256, 128, 3)
    pair = lib.ffn_quant_manifest_find_pair(h, b"mlpGateUp", 0)
    assert pair >= 0 and lib.ffn_quant_manifest_find_pair(h, b"mlpGateUp", 7) < 0
    lib.ffn_quant_manifest_pair_shape(h, pair, ctypes.byref(n), ctypes.byref(k), ctypes.byref(g))
    assert (n.value, k.value) == (512, 256)
    lib.ffn_quant_manifest_free(h)


MUTANTS = [
    ("a version this reader does not speak", '"manifest_version": 1', '"manifest_version": 2', FORMAT),
    ("a qmin that is not the frozen one", '"qmin": -7', '"qmin": -6', FORMAT),
    ("a foreign group", '"group": 128,\n      "group_axis"', '"group": 64,\n      "group_axis"', SHAPE),
    ("a K that is not a whole number of groups", '"logical_shape": [\n        256,\n        256\n      ]',
     '"logical_shape": [\n        256,\n        192\n      ]', SHAPE),
    ("a group axis that is not K", '"group_axis": "k"', '"group_axis": "n"', FORMAT),
    ("packed bytes that disagree with the shape", '"bytes": 32768', '"bytes": 32769', SHAPE),
    ("a scale count that disagrees with the shape", '"count": 512', '"count": 511', SHAPE),
    ("a packed dtype that is not u8", '"dtype": "u8"', '"dtype": "f16"', FORMAT),
    ("an entry with no int4 precision cell", '"precision": "int4"', '"precision": "bf16"', SHAPE),
    ("a pair whose rows are not its members'", '"logical_shape": [\n        512,\n        256\n      ]',
     '"logical_shape": [\n        511,\n        256\n      ]', SHAPE),
    ("a pair member that is not an entry", '"role": "mlpUp"', '"role": "mlpDown"', SHAPE),
    ("a duplicate key", '"manifest_version": 1', '"manifest_version": 1,\n  "manifest_version": 1', SYNTAX),
    ("a missing required section", '"entries":', '"entries_x":', SYNTAX),
]


@pytest.mark.parametrize("label,needle,replacement,want", MUTANTS, ids=[m[0] for m in MUTANTS])
def test_refusals(fixture_text, label, needle, replacement, want):
    assert needle in fixture_text, "the anchor is not in the fixture"
    mutant = fixture_text.replace(needle, replacement, 1)
    st, _ = parse(mutant)
    assert st == want, (label, L.load().ffn_int4_last_error())
    ref = ref_parse_status(mutant)
    assert ref in (None, want), f"the reference reader answers {ref}"


def test_more_refusals(fixture_text):
    at = fixture_text.index('"sha256": "', fixture_text.index("artifacts/mlpGate_layer0.packed") - 200)
    # corrupt the digest recorded for the gate payload: one character, same length
    anchor = fixture_text.index("artifacts/mlpGate_layer0.packed")
    at = fixture_text.index('"sha256": "', anchor) + len('"sha256": "')
    bad = fixture_text[:at] + "z" + fixture_text[at + 1:]
    assert parse(bad)[0] == FORMAT and ref_parse_status(bad) in (None, FORMAT)
    for doc in (fixture_text[:-20], "", "[]", fixture_text + "x"):
        assert parse(doc)[0] == SYNTAX
        assert ref_parse_status(doc) in (None, SYNTAX)


def test_artifact_read(tmp_path):
    lib = L.load()
    payload = bytes((i * 7 + 1) & 0xFF for i in range(64))
    (tmp_path / "one.packed").write_bytes(payload)
    digest = hashlib.sha256(payload).hexdigest().encode()
    out, n = ctypes.c_void_p(), ctypes.c_size_t()

    def read(file=b"one.packed", dtype=b"u8", size=64, want=b"u8"):
        return lib.ffn_quant_artifact_read(str(tmp_path).encode(), file, dtype, size, digest, want,
                                           ctypes.byref(out), ctypes.byref(n))
    assert read() == OK and n.value == 64
    assert ctypes.string_at(out, 64) == payload
    lib.ffn_host_free(out)
    corrupted = bytearray(payload)
    corrupted[3] ^= 0xFF
    (tmp_path / "one.packed").write_bytes(bytes(corrupted))
    assert read() == HASH and not out.value                 # a refused read hands back no buffer
    assert read(size=65) == IO                              # size is checked before the digest
    assert read(want=b"bf16") == FORMAT
    assert read(file=b"two.packed") == IO
    (tmp_path / "one.packed").write_bytes(payload)
    assert read(dtype=b"anything", want=None) == OK         # no expectation, no dtype check (csrc/quant_manifest.c:1095)
    lib.ffn_host_free(out)


def test_shard_views():
    lib = L.load()
    v = (ctypes.c_longlong * 4)()
    assert lib.ffn_shard_view(1, 16, 8, 2, 1, v) == 0 and list(v) == [8, 8, 0, 8]     # MLP_UP [16,8] rank 1 of 2
    assert lib.ffn_shard_view(2, 8, 16, 2, 1, v) == 0 and list(v) == [0, 8, 8, 8]     # MLP_DOWN [8,16] rank 1
    assert lib.ffn_shard_view(1, 16, 8, 1, 0, v) == 0 and list(v) == [0, 16, 0, 8]    # tp 1: the whole tensor
    assert lib.ffn_shard_view(1, 16, 8, 2, 2, v) == -4                                # rank out of range
    assert lib.ffn_shard_view(1, 15, 8, 2, 0, v) == -4                                # uneven split
    assert b"does not divide" in lib.ffn_int4_last_error()
