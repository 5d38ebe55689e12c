"""Differential check of the strict manifest reader against the reference's own reader
(csrc/quant_manifest.c, compiled into oracle/_ref): a valid manifest is damaged in one place at a time -
a field deleted, retyped, resized, renamed or given an out-of-range value, or the text cut short - and
both readers must return the same QuantManifestStatus (OK, ARG, SYNTAX, FORMAT, SHAPE) for every one of
them.  Skipped where the reference's sources were not available to build oracle/_ref."""
import copy
import ctypes
import random

import pytest

from haskell_infer_demo_b200 import lib as L
from oracle import ffn_oracle as o
import sidecar_util

VALUES = [0, 1, -1, 2, 7, 8, 127, 128, 129, 256, -7, -8, 2 ** 31, 2 ** 40, 1.5, 128.0, "", "u8", "bf16", "int4", "k",
          "mlpGate", "mlpUp", "mlpDown", "x" * 63, "x" * 64, "x" * 70, "p" * 511, "p" * 512, "a" * 64, "A" * 64, "g" * 64,
          "a" * 65, None, True, [], {}, [1, 2], [384, 256], [384, 256, 1], {"role": "mlpGate"}]


def paths(node, prefix=()):
    out = []
    if isinstance(node, dict):
        for k, v in node.items():
            out.append(prefix + (k,))
            out += paths(v, prefix + (k,))
    elif isinstance(node, list):
        for i, v in enumerate(node):
            out.append(prefix + (i,))
            out += paths(v, prefix + (i,))
    return out


def parent(doc, path):
    for k in path[:-1]:
        doc = doc[k]
    return doc


@pytest.fixture(scope="module")
def readers():
    ref = o.ref_lib("libref_quant_manifest.so")
    if ref is None:
        pytest.skip("oracle/_ref was not built (no reference checkout)")
    ref.quant_manifest_parse.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    scratch = ctypes.create_string_buffer(2 << 20)          # struct QuantManifest is about 1 MiB
    lib = L.load()

    def ours(text):
        handle = ctypes.c_void_p()
        st = lib.ffn_quant_manifest_parse(text.encode(), ctypes.byref(handle))
        if st == 0:
            lib.ffn_quant_manifest_free(handle)
        return st

    return ours, lambda text: ref.quant_manifest_parse(text.encode(), scratch, None, 0)


def test_one_fault_at_a_time_gets_the_references_status(readers, tmp_path):
    ours, theirs = readers
    _, layers = o.draw_config(256, 384, 21, layers=2)
    base = sidecar_util.manifest_dict(str(tmp_path), layers)
    rng = random.Random(20240607)
    seen = {}
    for case in range(900):
        doc = copy.deepcopy(base)
        path = rng.choice(paths(doc))
        where, last = parent(doc, path), path[-1]
        kind = rng.random()
        if kind < 0.25:
            del where[last]
        elif kind < 0.80:
            where[last] = rng.choice(VALUES)
        elif kind < 0.90 and isinstance(where, dict):
            where[last + rng.choice(["x", "_", "y" * 60, "z" * 600])] = where.pop(last)      # renamed (and maybe oversized) key
        elif isinstance(where[last], int) and not isinstance(where[last], bool):
            where[last] += rng.choice([-1, 1, 2, 128, -10 ** 6])
        elif isinstance(where[last], str):
            where[last] = where[last][:-1] if rng.random() < 0.5 else where[last] + "f"
        elif isinstance(where[last], list) and where[last]:
            where[last] = where[last] + [copy.deepcopy(where[last][0])]
        text = sidecar_util.dumps(doc)
        a, b = ours(text), theirs(text)
        assert a == b, f"case {case}: {path} -> ours {a}, reference {b}: {L.load().ffn_int4_last_error().decode()}"
        seen[a] = seen.get(a, 0) + 1
    assert set(seen) == {0, 1, 2, 3, 4}, seen                  # every status class was exercised
    whole = sidecar_util.dumps(base)
    for case in range(200):                                  # a document cut short anywhere is a syntax error for both
        cut = whole[:rng.randrange(len(whole) - 1)]
        assert ours(cut) == theirs(cut) == 2
    for tail in (" ", "\n\n", "x", "{}", ","):
        assert ours(whole + tail) == theirs(whole + tail)
