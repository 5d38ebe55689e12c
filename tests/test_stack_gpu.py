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
from gpu_util import assert_ffn_close, dev_bf16, dev_bits, host_f32, upload_layer

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


def load_stack_golden():
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "stack_cfg4.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/stack_cfg4.npz has not been generated (tests/golden/make_stack_golden.py)")
    return np.load(path)


def check_stack_against_golden(dev, mlps, golden, comm=None, sync=None, what=""):
    """Teacher-forced and free-running gates of the 64-layer 27B-shape stack for one rank's operands
    `mlps` (shared by the single-GPU test and the tensor-parallel worker).  `sync` is called before every
    launch that other ranks must join within the kernels' bounded waits."""
    from haskell_infer_demo_b200 import synth
    nl, hidden, inter, tokens8, seed = [int(v) for v in golden["shape"]]
    sync = sync or (lambda: None)
    x8 = synth.stack_input_torch(seed, tokens8, hidden, dev)
    tok0 = o.bf16_to_f32(golden["tok0_states"])
    tok0_y = o.bf16_to_f32(golden["tok0_ffn_out"])

    def one_layer(l, h_in, y_want, label):
        """Layer l from the oracle's input state.  The residual stream of this synthetic model grows
        (|h| ~ 100 after 64 layers, one BF16 ulp of h then being larger than any error in y), so the
        gate is on the FFN output y at the FFN bars, and the state must be exactly bf16(h_in + y) for
        the y the device produced."""
        h = h_in.clone()
        y = torch.empty_like(h)
        sync()
        decode_stack([mlps[l]], h, comm=comm, layer_out=y)
        L.device_status()
        rel = assert_ffn_close(host_f32(y), y_want, label)[1]
        assert np.array_equal(host_f32(h), o.residual_add(host_f32(h_in), host_f32(y))), f"{label}: h is not bf16(h + y)"
        return rel

    # (i) teacher-forced, one token, every layer: input = the oracle's state before the layer
    worst = 0.0
    for l in range(nl):
        h_in = x8[:1] if l == 0 else dev_bf16(tok0[l - 1:l], dev)
        worst = max(worst, one_layer(l, h_in, tok0_y[l:l + 1], f"{what} layer {l} teacher-forced, M=1"))
    # eight tokens on the kept layers
    for j, l in enumerate(int(v) for v in golden["m8_layers"]):
        one_layer(l, dev_bits(golden["m8_states"][j, 0], dev), o.bf16_to_f32(golden["m8_ffn_out"][j]),
                  f"{what} layer {l} teacher-forced, M=8")
    # (ii) free-running final state against the oracle-vs-oracle spread
    spread = float(golden["spread_rel_l2"])
    want = o.bf16_to_f32(golden["final_f64"])
    out = {}
    for m in (1, 8):
        h = x8[:m].clone()
        sync()
        decode_stack(mlps, h, comm=comm)
        L.device_status()
        rel = o.compare(host_f32(h), want[:m])[1]
        out[m] = (rel, h)
        print(f"{what} 64-layer stack M={m}: free-running rel-L2 {rel:.3g} (FP32- vs FP64-accumulating CPU oracles: {spread:.3g}); "
              f"worst teacher-forced layer rel-L2 {worst:.3g}")
        assert rel <= max(5e-3, 2 * spread)
    return out


@pytest.mark.parametrize("kmajor", [False, True])
def test_stack_27b_shape_64_layers_against_golden(cuda, kmajor):
    """BASELINE configs[4] at its full shape on one GPU: 64 independently generated layers (H=5120,
    I=17408), checked against the committed CPU-oracle trajectory - layer by layer through the row-major
    kernel, and with k-major copies registered (one persistent launch for the whole stack at M=1)."""
    from haskell_infer_demo_b200 import synth
    golden = load_stack_golden()
    nl, hidden, inter, _, seed = [int(v) for v in golden["shape"]]
    mlps = [synth.stack_layer_torch(seed, l, hidden, inter, 1, 0, cuda) for l in range(nl)]
    # the device-side generator and quantizer reproduce the CPU side's bytes
    import hashlib
    t = mlps[0].tensors
    got = ",".join(hashlib.sha256(a.cpu().numpy().tobytes()).hexdigest() for a in (t[0], t[1].view(torch.int16), t[2], t[3].view(torch.int16)))
    assert got == str(golden["digest_layer0"])
    if kmajor:
        for m in mlps:
            m.prepare()
    check_stack_against_golden(cuda, mlps, golden, what="TP=1" + (" k-major" if kmajor else ""))
