"""The GPU quantizer (ffn_quantize_int4) against the reference's: the known-answer vectors of the
reference's format gate (tests/quantization_format_test.c), its deterministic [8,256] fixture, and
the SHA-256 digests of the seeded configurations' artifacts as the reference's compiled quantizer
made them (tests/golden/config_digests.json).  Byte identity throughout."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200 import ops
from oracle import ffn_oracle as o

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def quantize_gpu(w, cuda):
    """FP32 [N, K] numpy -> (status, packed u8 [N, K/2], scales u16 [N, K/128]) through the C ABI."""
    n, k = w.shape
    wd = torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32)).to(cuda)
    packed = torch.full((n, max(k // 2, 1)), 0xAB, dtype=torch.uint8, device=cuda)
    scales = torch.full((n, max(k // 128, 1)), 0x1234, dtype=torch.int16, device=cuda)
    st = L.load().ffn_quantize_int4(wd.data_ptr(), packed.data_ptr(), scales.data_ptr(), n, k, None)
    return st, packed.cpu().numpy(), scales.cpu().numpy().view(np.uint16)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_known_byte_pattern_and_clip(cuda):
    """Codes {0,1,-1,-7,7,3,-3,2} at scale exactly 1.0 pack to 10 9F 37 2D
    (quantization_format_test.c:118-153); +-0.7000001 against scale 0.1 clips to +-7 (:194-201); an
    all-zero group gets scale 1.0 and zero bytes (:183-190)."""
    w = np.zeros((8, 256), np.float32)
    w[0, :8] = [0, 1, -1, -7, 7, 3, -3, 2]
    w[1, :4] = [0.7, 0.7000001, -0.7000001, 0.35]
    st, packed, scales = quantize_gpu(w, cuda)
    assert st == 0
    assert packed[0, :4].tolist() == [0x10, 0x9F, 0x37, 0x2D]
    assert scales[0, 0] == 0x3F80 and scales[0, 1] == 0x3F80       # 7/7, and the all-zero second group
    assert not packed[0, 4:].any() and not packed[2:].any()
    want_p, want_s = o.quantize(w)
    assert np.array_equal(packed, want_p) and np.array_equal(scales, want_s)


def test_reference_fixture(cuda):
    """The reference's deterministic [8,256] fixture, emitted by the reference binary."""
    with open(os.path.join(GOLDEN, "format_fixture.json")) as f:
        fx = json.load(f)
    w = np.array(fx["weights_f32_bits"], np.uint32).view(np.float32).reshape(fx["n"], fx["k"])
    st, packed, scales = quantize_gpu(w, cuda)
    assert st == 0
    assert packed.ravel().tolist() == fx["packed"]
    assert scales.ravel().tolist() == fx["scales_bf16"]


@pytest.mark.parametrize("cfg", [0, 1])
def test_config_digests(cuda, cfg):
    """The seeded configurations, quantized on the GPU, hash to what the reference's quantizer wrote."""
    with open(os.path.join(GOLDEN, "config_digests.json")) as f:
        want = json.load(f)[str(cfg)]
    h, i = want["hidden"], want["inter"]
    rng = np.random.default_rng(want["seed"])
    rng.standard_normal((1, h), dtype=np.float32)                  # the activations come first in the draw order
    for name, shape in (("gate", (i, h)), ("up", (i, h)), ("down", (h, i))):
        w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        st, packed, scales = quantize_gpu(w, cuda)
        assert st == 0
        assert sha(packed) == want[f"{name}_packed_sha256"], name
        assert sha(scales) == want[f"{name}_scales_sha256"], name


def test_requantizing_the_dequantized_weights_is_a_fixed_point(cuda):
    """quantization_format_test.c:228-237."""
    rng = np.random.default_rng(5)
    w = rng.standard_normal((64, 512), dtype=np.float32) * np.float32(0.05)
    st, packed, scales = quantize_gpu(w, cuda)
    assert st == 0
    deq = o.dequantize(packed, scales)
    st2, packed2, scales2 = quantize_gpu(deq, cuda)
    assert st2 == 0 and np.array_equal(packed, packed2) and np.array_equal(scales, scales2)


def test_refusals_leave_the_outputs_untouched(cuda):
    """Non-finite elements, a group that rounds to a zero scale (1e-40, :205-209) and shapes the
    format cannot hold are refused before anything is written."""
    lib = L.load()
    base = np.random.default_rng(6).standard_normal((8, 256), dtype=np.float32)
    for bad, needle in ((np.nan, "element 300 is not finite"), (np.inf, "element 300 is not finite")):
        w = base.copy()
        w.ravel()[300] = bad
        w.ravel()[900] = bad                                     # the first offender is the one named
        st, packed, scales = quantize_gpu(w, cuda)
        assert st == -3 and needle in lib.ffn_int4_last_error().decode()
        assert (packed == 0xAB).all() and (scales == 0x1234).all()
    w = base.copy()
    w[3, 128:] = np.float32(1e-40)
    st, packed, scales = quantize_gpu(w, cuda)
    assert st == -3 and "row 3 group 1" in lib.ffn_int4_last_error().decode()
    assert (packed == 0xAB).all() and (scales == 0x1234).all()
    assert quantize_gpu(np.zeros((8, 192), np.float32), cuda)[0] == -4     # K is not a whole number of groups
    assert quantize_gpu(np.zeros((12, 256), np.float32), cuda)[0] == -4    # N is not a multiple of the row tile
