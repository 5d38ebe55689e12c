"""ffn_load_quantized_ffn on a GPU: a sidecar written in the converter's layout is read, verified,
sliced per rank with the global scales and uploaded; the device bytes equal the oracle's slices and the
FFN computed from the loaded operands matches the oracle.  Refusals follow
tests/test_quantized_sharding.py:99-119 (mid-group split) and tests/test_quantized_ffn.py:332-362
(corrupted payload)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200.lib import MlpWeights
from haskell_infer_demo_b200.ops import DenseMlp
from oracle import ffn_oracle as o
from gpu_util import assert_ffn_close, dev_bf16, host_f32
import sidecar_util

pytestmark = pytest.mark.gpu


def load(root, layers, h, i, tp, rank):
    handle = ctypes.c_void_p()
    st = L.load().ffn_load_quantized_ffn(str(root).encode(), layers, h, i, tp, rank, ctypes.byref(handle))
    return st, handle


def device_bytes(ptr, nbytes):
    """Raw device bytes at `ptr` (a pointer the loader owns) as a numpy array."""
    out = np.empty(nbytes, np.uint8)
    torch.cuda.synchronize()
    cudart = ctypes.CDLL("libcudart.so.12")   # the runtime torch already loaded
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    assert cudart.cudaMemcpy(out.ctypes.data, ptr, nbytes, 2) == 0   # 2 = cudaMemcpyDeviceToHost
    return out


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_load_slices_and_runs(cuda, tmp_path, tp):
    lib = L.load()
    h, i, nl = 512, 1024, 2
    x, layers = o.draw_config(h, i, 17, layers=nl)
    sidecar_util.write_sidecar(str(tmp_path), layers)
    partial_sum = [np.zeros((1, h), np.float64) for _ in range(nl)]
    for rank in range(tp):
        st, handle = load(tmp_path, nl, h, i, tp, rank)
        assert st == 0, lib.ffn_int4_last_error()
        for l in range(nl):
            w = MlpWeights()
            assert lib.ffn_quantized_ffn_layer(handle, l, ctypes.byref(w)) == 0
            gp, gs, dp, ds = o.slice_rank(layers[l].gate_up_packed, layers[l].gate_up_scales, layers[l].down_packed,
                                          layers[l].down_scales, tp, rank)
            assert np.array_equal(device_bytes(w.gate_up_i4, gp.size), gp.ravel())
            assert np.array_equal(device_bytes(w.gate_up_i4_scales, gs.size * 2), gs.ravel().view(np.uint8))
            assert np.array_equal(device_bytes(w.down_i4, dp.size), dp.ravel())
            assert np.array_equal(device_bytes(w.down_i4_scales, ds.size * 2), ds.ravel().view(np.uint8))
            assert lib.ffn_decode_layer_is_prepared(ctypes.byref(w)) == 0      # k-major copies are an opt-in (below)
            if tp == 1:
                # run the FFN straight from the loaded operands
                dims = L.ModelDims()
                dims.hidden_size, dims.intermediate_size, dims.max_chunk = h, i, 128
                xd = dev_bf16(x, cuda)
                ws = torch.empty(h + 3 * i, dtype=torch.bfloat16, device=cuda)
                out = torch.empty((1, h), dtype=torch.bfloat16, device=cuda)
                L.check(lib.ffn_forward_mlp_prepared(None, None, ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(ws.data_ptr()),
                                                     ctypes.c_void_p(out.data_ptr()), ctypes.byref(w), 1, ctypes.byref(dims)))
                L.device_status()
                assert_ffn_close(host_f32(out), o.ffn(layers[l], x), f"layer {l} from the loaded sidecar")
        if tp == 1:
            # the opt-in k-major copies for the whole handle: another kernel, the same answer
            assert lib.ffn_quantized_ffn_prepare_decode(handle) == 0, lib.ffn_int4_last_error()
            for l in range(nl):
                w = MlpWeights()
                assert lib.ffn_quantized_ffn_layer(handle, l, ctypes.byref(w)) == 0
                assert lib.ffn_decode_layer_is_prepared(ctypes.byref(w)) == 1
                L.check(lib.ffn_forward_mlp_prepared(None, None, ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(ws.data_ptr()),
                                                     ctypes.c_void_p(out.data_ptr()), ctypes.byref(w), 1, ctypes.byref(dims)))
                L.device_status()
                assert_ffn_close(host_f32(out), o.ffn(layers[l], x), f"layer {l} through its k-major copy")
        assert lib.ffn_quantized_ffn_free(handle) == 0


def test_refusals(cuda, tmp_path):
    lib = L.load()
    # a tp=2 split of intermediate=384 lands inside a group (tests/test_quantized_sharding.py:99-119)
    x, layers = o.draw_config(256, 384, 5, layers=1)
    root = tmp_path / "mid"
    root.mkdir()
    sidecar_util.write_sidecar(str(root), layers)
    st, _ = load(root, 1, 256, 384, 1, 0)
    assert st == 0
    st, _ = load(root, 1, 256, 384, 2, 1)
    assert st == -3 and b"splits K at a non-group boundary" in lib.ffn_int4_last_error()
    # the sidecar must cover every dense layer
    st, _ = load(root, 2, 256, 384, 1, 0)
    assert st == -3 and b"covers 1 of 2 dense layers" in lib.ffn_int4_last_error()
    # a shape that is not the checkpoint's
    st, _ = load(root, 1, 256, 512, 1, 0)
    assert st == -3 and b"mlpGateUp pair is" in lib.ffn_int4_last_error()
    # a corrupted payload is a hash refusal, and nothing stays loaded
    path = root / "artifacts" / "mlpDown_layer0.packed"
    raw = bytearray(path.read_bytes())
    raw[7] ^= 0x55
    path.write_bytes(bytes(raw))
    st, _ = load(root, 1, 256, 384, 1, 0)
    assert st == -3 and b"hashes to" in lib.ffn_int4_last_error()
    # a missing sidecar
    st, _ = load(tmp_path / "absent", 1, 256, 384, 1, 0)
    assert st == -3 and b"cannot open" in lib.ffn_int4_last_error()
