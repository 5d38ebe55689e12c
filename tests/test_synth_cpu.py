"""The counter-based synthetic weights are the same bits in numpy and in torch, whole or sliced, so
the CPU oracle's golden trajectory and the GPU tests' device-generated operands describe one model."""
import numpy as np
import torch

from haskell_infer_demo_b200 import synth


def test_numpy_and_torch_agree_bit_for_bit():
    for tensor, sigma in ((synth.W_GATE, 0.02), (synth.W_DOWN, 0.02), (synth.X, 1.0), (synth.W_NORM, 0.1)):
        a = synth.matrix_numpy(4, tensor, 7, 300, 640, sigma, row_block=128)
        b = synth.matrix_torch(4, tensor, 7, 300, 640, sigma, "cpu", row_block=77).numpy()
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    whole = synth.matrix_numpy(4, synth.W_DOWN, 2, 256, 1024, 0.02)
    part = synth.matrix_torch(4, synth.W_DOWN, 2, 256, 1024, 0.02, "cpu", row_off=8, nrows=100, col_off=384, ncols=256).numpy()
    assert np.array_equal(part, whole[8:108, 384:640])


def test_streams_differ_and_look_normal():
    a = synth.matrix_numpy(4, synth.W_GATE, 0, 512, 1024, 0.02)
    b = synth.matrix_numpy(4, synth.W_GATE, 1, 512, 1024, 0.02)
    c = synth.matrix_numpy(4, synth.W_UP, 0, 512, 1024, 0.02)
    d = synth.matrix_numpy(5, synth.W_GATE, 0, 512, 1024, 0.02)
    for other in (b, c, d):
        assert abs(np.corrcoef(a.ravel(), other.ravel())[0, 1]) < 0.01
    assert abs(a.std() - 0.02) < 2e-4 and abs(a.mean()) < 1e-4
    assert np.abs(a).max() <= 0.02 * 3.47


def test_a_column_slice_quantizes_to_the_whole_tensors_bytes():
    """What lets a rank quantize only its own down columns: groups never straddle a 128-aligned split."""
    from oracle import ffn_oracle as o
    w = synth.matrix_numpy(4, synth.W_DOWN, 0, 64, 1024, 0.02)
    p, s = o.quantize(w)
    ps, ss = o.quantize(np.ascontiguousarray(w[:, 256:512]))
    assert np.array_equal(ps, p[:, 128:256]) and np.array_equal(ss, s[:, 2:4])
