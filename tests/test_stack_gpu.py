"""Config-4 style stack on the GPU: h <- h + FFN_l(GemmaRMSNorm_l(h)) with identity mixers, through
ffn_decode_stack.  Two gates, as the deep stack is chaotic under BF16 rounding (one rounding that falls
differently decorrelates the residual stream after a few dozen layers):
  (i)  teacher-forced, per layer: every layer is fed the oracle's input for that layer and must meet
       the FFN bars (relative L2 <= 5e-3, max-abs <= max(2e-2, one BF16 ulp));
  (ii) free-running: the final state must stay within twice the spread between two legitimate CPU
       oracles (FP64- vs FP32-accumulating) on the same data, or the per-FFN bar, whichever is larger.
"""
import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200.ops import decode_stack
from oracle import ffn_oracle as o
from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,nlayers", [(1, 12), (2, 6), (8, 6)])
def test_stack_teacher_forced_and_free_running(cuda, tokens, nlayers):
    hidden, inter = 1024, 3072
    h0, layers = o.draw_config(hidden, inter, 4, tokens=tokens, layers=nlayers, with_norm=True)
    ref64 = o.stack(layers, h0)                         # free-running oracle, FP64 accumulation
    ref32 = o.stack(layers, h0, accumulate="f32")       # a second legitimate oracle
    mlps = [upload_layer(lay, cuda, with_norm=True) for lay in layers]

    # (i) teacher-forced: layer l from the oracle's h_{l-1}
    inputs = [h0] + ref64[:-1]
    for l in range(nlayers):
        h = dev_bf16(inputs[l], cuda).clone()
        decode_stack([mlps[l]], h)
        L.device_status()
        assert_ffn_close(host_f32(h), ref64[l], f"layer {l} teacher-forced, M={tokens}")

    # (ii) free-running through all layers in one call
    h = dev_bf16(h0, cuda).clone()
    decode_stack(mlps, h)
    L.device_status()
    got = host_f32(h)
    _, spread = o.compare(ref32[-1], ref64[-1])
    _, rel = o.compare(got, ref64[-1])
    print(f"M={tokens} L={nlayers}: free-running rel-L2 {rel:.3g}; oracle-vs-oracle spread {spread:.3g}")
    assert rel <= max(5e-3, 2 * spread)

    # the one-call stack equals the layer-by-layer composition bit for bit (nothing is carried in
    # hidden state between layers)
    h2 = dev_bf16(h0, cuda).clone()
    for m in mlps:
        decode_stack([m], h2)
    L.device_status()
    assert torch.equal(h2.view(torch.int16), h.view(torch.int16))


def test_stack_refusals(cuda):
    from haskell_infer_demo_b200.lib import FfnError
    h0, layers = o.draw_config(256, 512, 1, layers=1, with_norm=False)
    mlp = upload_layer(layers[0], cuda)            # no post-norm weight
    with pytest.raises(FfnError, match="post-norm"):
        decode_stack([mlp], dev_bf16(h0, cuda).clone())
