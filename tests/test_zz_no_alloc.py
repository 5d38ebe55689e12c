"""The allocation-free FFN entry point (ffn_forward_mlp_prepared_noalloc), through the C ABI.

Some users of this library cannot let it allocate device memory: their process gives the whole GPU
to its own memory arena when it starts (so a cudaMalloc issued by a library fails), or their decode
loop cannot afford the device-wide synchronisation that cudaMalloc and cudaFree bring.  For them the
fused kernel's scratch lives in a fixed array inside the library.  This test calls that entry point
twice in a row - the array keeps the previous call's contents, so the second call is the interesting
one - and checks both outputs against the ordinary entry point's on the same inputs.  It also checks
that a request beyond the array's stated size is refused.  The file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from oracle import ffn_oracle as o
from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer

pytestmark = pytest.mark.gpu


def _call_noalloc(mlp, x, out):
    lib = L.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.ffn_forward_mlp_prepared_noalloc(stream, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                                ctypes.byref(mlp.weights), x.shape[0], ctypes.byref(mlp.dims))


@pytest.mark.parametrize("hidden,inter,tokens", [(1024, 3072, 1), (1024, 3072, 2), (2560, 9728, 1)])
def test_noalloc_matches_regular_entry_point_twice(cuda, hidden, inter, tokens):
    x, layers = o.draw_config(hidden, inter, 21, tokens=tokens)
    want = o.ffn(layers[0], x)
    mlp = upload_layer(layers[0], cuda)
    xd = dev_bf16(x, cuda)
    regular = mlp.forward_mlp_prepared(xd)
    L.device_status()
    # second input, so the second call cannot pass by finding the first call's result in place
    x2 = o.bf16_round(-0.5 * x + 0.25)
    xd2 = dev_bf16(x2, cuda)
    regular2 = mlp.forward_mlp_prepared(xd2)
    L.device_status()

    out1 = torch.full_like(regular, float("nan"))
    out2 = torch.full_like(regular, float("nan"))
    before = torch.cuda.memory_allocated()
    assert _call_noalloc(mlp, xd, out1) == 0, L.load().ffn_int4_last_error()
    assert _call_noalloc(mlp, xd2, out2) == 0, L.load().ffn_int4_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    # same kernel, same arithmetic: the tolerance of the FFN tests, and in fact the same bits
    assert_ffn_close(host_f32(out1), host_f32(regular), "no-alloc call 1 vs regular entry point")
    assert_ffn_close(host_f32(out2), host_f32(regular2), "no-alloc call 2 vs regular entry point")
    assert torch.equal(out1.view(torch.int16), regular.view(torch.int16))
    assert torch.equal(out2.view(torch.int16), regular2.view(torch.int16))
    assert_ffn_close(host_f32(out1), want, "no-alloc vs oracle")


def test_noalloc_refuses_sizes_beyond_its_array(cuda):
    lib = L.load()
    x, layers = o.draw_config(256, 512, 3)
    mlp = upload_layer(layers[0], cuda)
    xd = dev_bf16(x, cuda)
    out = torch.empty((1, 256), dtype=torch.bfloat16, device=cuda)
    mlp.dims.intermediate_size = 65536 + 128        # one token, more act elements than the array holds
    assert _call_noalloc(mlp, xd, out) == -4
    assert b"exceeds the static scratch" in lib.ffn_int4_last_error()
    mlp.dims.intermediate_size = 512
    x3 = torch.zeros((3, 256), dtype=torch.bfloat16, device=cuda)
    out3 = torch.empty((3, 256), dtype=torch.bfloat16, device=cuda)
    assert _call_noalloc(mlp, x3, out3) == -4       # three tokens: not a shape this entry point takes
    assert _call_noalloc(mlp, xd, out) == 0         # and it still works afterwards
    torch.cuda.synchronize()
