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


@pytest.mark.parametrize("hidden,inter,tokens", [(1024, 3072, 1), (1024, 3072, 2), (2560, 9728, 1), (5120, 17408, 1)])
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
    # both calls completed: the entry point's own status word (inside the static array) reads clean
    assert L.load().ffn_int4_noalloc_status(None, None) == 0, L.load().ffn_int4_last_error()


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


_FRESH_PROCESS = r"""
import ctypes, sys
import torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from haskell_infer_demo_b200 import lib as L
from oracle import ffn_oracle as o
from gpu_util import dev_bf16, host_f32, upload_layer, assert_ffn_close
cuda = torch.device("cuda", 0)
x, layers = o.draw_config(1024, 3072, 21)
mlp = upload_layer(layers[0], cuda)
xd = dev_bf16(x, cuda)
out = torch.full((1, 1024), float("nan"), dtype=torch.bfloat16, device=cuda)
torch.cuda.synchronize()
lib = L.load()
def call():
    return lib.ffn_forward_mlp_prepared_noalloc(None, ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                                ctypes.byref(mlp.weights), 1, ctypes.byref(mlp.dims))
# the very first call into the library in this process: symbol lookup and kernel attributes on a cold context
assert call() == 0, lib.ffn_int4_last_error()
assert lib.ffn_int4_noalloc_status(None, None) == 0, lib.ffn_int4_last_error()
free0 = torch.cuda.mem_get_info()[0]          # cudaMemGetInfo: sees every allocation of the process, not only torch's
for _ in range(20):
    assert call() == 0
assert lib.ffn_int4_noalloc_status(None, None) == 0
assert torch.cuda.mem_get_info()[0] == free0, "device memory was allocated by an allocation-free call"
got = host_f32(out).copy()
assert_ffn_close(got, o.ffn(layers[0], x), "no-alloc entry as the first call of a process")
regular = mlp.forward_mlp_prepared(xd)        # the ordinary entry point (this one does allocate its words)
L.device_status()
assert torch.equal(regular.view(torch.int16), out.view(torch.int16))
print("fresh-process no-alloc ok")
"""


def test_noalloc_is_allocation_free_as_first_call_of_a_fresh_process(cuda):
    """The stated use: a process whose first and only calls into the library are the allocation-free
    entry point and its status reader.  Run in a child process so that nothing else has touched the
    library; the free device memory the driver reports (cudaMemGetInfo, which also sees a cudaMalloc
    made inside a library) must not move across twenty calls."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-c", _FRESH_PROCESS, root], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "fresh-process no-alloc ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]
