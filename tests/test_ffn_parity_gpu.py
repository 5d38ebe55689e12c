"""GPU parity of the FFN operator (ffn_forward_mlp through the C ABI) against the CPU oracle on the
seeded configurations, plus the committed golden output of config 0."""
import json
import os

import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from oracle import ffn_oracle as o
from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def drawn():
    cache = {}

    def get(cfg, tokens):
        if (cfg, tokens) not in cache:
            spec = o.CONFIGS[cfg]
            x, layers = o.draw_config(spec["hidden"], spec["inter"], spec["seed"], tokens=tokens)
            cache[(cfg, tokens)] = (x, layers[0], o.ffn(layers[0], x))
        return cache[(cfg, tokens)]
    return get


@pytest.mark.parametrize("fused", [1, 0])
@pytest.mark.parametrize("cfg,tokens", [(0, 1), (0, 2), (0, 3), (0, 4), (0, 8), (0, 16), (0, 33), (0, 64), (0, 100),
                                        (1, 1), (1, 2), (1, 8), (1, 64), (2, 1), (2, 2), (2, 16)])
def test_ffn_matches_oracle(cuda, drawn, cfg, tokens, fused):
    """Single-launch fused kernel (M <= 2), the tensor-core pair (3 <= M, blocks of 64) and the
    three-kernel generic route (fused=0) against the CPU oracle."""
    if not fused and tokens > 8:
        pytest.skip("the generic route is covered up to M=8 here and up to M=64 by the kernel gate")
    x, layer, want = drawn(cfg, tokens)
    mlp = upload_layer(layer, cuda)
    old = L.load().ffn_int4_set_fused(fused)
    try:
        got = host_f32(mlp.forward_mlp_prepared(dev_bf16(x, cuda)))
        L.device_status()
    finally:
        L.load().ffn_int4_set_fused(old)
    max_abs, rel = assert_ffn_close(got, want, f"config {cfg} M={tokens} fused={fused}")
    print(f"config {cfg} M={tokens} fused={fused}: max-abs {max_abs:.3g} rel-L2 {rel:.3g}")


def test_fused_is_deterministic_and_repeatable(cuda, drawn):
    """Same inputs, many launches: bit-identical outputs (fixed-order reductions, self-resetting
    hand-over buffers) and the activation left in the workspace equals the oracle's within one ulp."""
    x, layer, want = drawn(1, 1)
    mlp = upload_layer(layer, cuda)
    xd = dev_bf16(x, cuda)
    ws = mlp.workspace(1)
    first = mlp.forward_mlp_prepared(xd, ws=ws).clone()
    for _ in range(20):
        again = mlp.forward_mlp_prepared(xd, ws=ws)
        assert torch.equal(first.view(torch.int16), again.view(torch.int16))
    L.device_status()
    _, gu, act = o.ffn(layer, x, intermediates=True)
    h, i = layer.hidden, layer.inter
    got_act = host_f32(ws[h + 2 * i:h + 3 * i].view(1, i))
    assert o.compare(got_act, act)[1] <= 5e-3


def test_fused_shapes_alternate(cuda, drawn):
    """Launches of different shapes and token counts follow each other on one device: the buffers
    that hand act from phase 1 to phase 2 must never show a later launch an earlier launch's values."""
    order = [(2, 2), (0, 1), (2, 1), (1, 2), (0, 2), (2, 2), (1, 1), (2, 1)]
    mlps = {key: upload_layer(drawn(*key)[1], cuda) for key in set(order)}   # the draw depends on the token count
    for cfg, tokens in order:
        x, _, want = drawn(cfg, tokens)
        got = host_f32(mlps[(cfg, tokens)].forward_mlp_prepared(dev_bf16(x, cuda)))
        L.device_status()
        assert_ffn_close(got, want, f"config {cfg} M={tokens} in a mixed sequence")


def test_config0_golden_output(cuda):
    """Against the committed fixture (made from weights the reference library quantized)."""
    with open(os.path.join(GOLDEN, "ffn_config0.json")) as f:
        fx = json.load(f)
    x, layers = o.draw_config(fx["hidden"], fx["inter"], fx["seed"])
    want = o.bf16_to_f32(np.array(fx["y_bf16"], np.uint16)).reshape(1, -1)
    mlp = upload_layer(layers[0], cuda)
    got = host_f32(mlp.forward_mlp_prepared(dev_bf16(x, cuda)))
    L.device_status()
    assert_ffn_close(got, want, "config 0 golden")


def test_forward_mlp_with_norm_and_workspace_layout(cuda):
    """forward_mlp applies the Gemma post-norm first and leaves the normalized activation at the
    start of the workspace, as the reference does (csrc/kernels/layers.cu:149-160)."""
    x, layers = o.draw_config(1024, 3072, 7, tokens=2, with_norm=True)
    lay = layers[0]
    normed = o.gemma_rmsnorm(x, lay.w_norm)
    want = o.ffn(lay, normed)
    mlp = upload_layer(lay, cuda, with_norm=True)
    ws = mlp.workspace(2)
    got = host_f32(mlp.forward_mlp(dev_bf16(x, cuda), ws=ws))
    torch.cuda.synchronize()
    ws_normed = host_f32(ws[:2 * 1024].view(2, 1024))
    assert np.allclose(ws_normed, normed, atol=1e-3, rtol=8e-3)
    assert_ffn_close(got, o.ffn(lay, ws_normed), "forward_mlp vs oracle on the device's own norm")
    assert o.compare(got, want)[1] <= 5e-3


def test_refusals(cuda):
    from haskell_infer_demo_b200.lib import FfnError
    x, layers = o.draw_config(256, 512, 1)
    mlp = upload_layer(layers[0], cuda)
    with pytest.raises(FfnError, match="max_chunk"):
        mlp.forward_mlp_prepared(torch.zeros((129, 256), dtype=torch.bfloat16, device=cuda))
    mlp.weights.gate_up_i4 = 0
    with pytest.raises(FfnError, match="no INT4 operands"):
        mlp.forward_mlp_prepared(dev_bf16(x, cuda))


@pytest.mark.parametrize("pinned", [True, False], ids=["pinned", "pageable"])
@pytest.mark.parametrize("tokens", [1, 2, 16])
def test_forward_mlp_host_matches_oracle(cuda, drawn, tokens, pinned):
    """The host-buffer entry (input and output in host memory, one call, synchronous): pinned buffers take
    the mapped paths (input fetched by a staging kernel, output written by the FFN kernel itself),
    pageable ones the copy calls; either way the result is complete when the call returns."""
    from haskell_infer_demo_b200.ops import bind_forward_mlp_host, forward_mlp_host
    x, layer, want = drawn(0, tokens)
    mlp = upload_layer(layer, cuda)
    h = o.CONFIGS[0]["hidden"]
    x_host = torch.from_numpy(o.bf16_bits(x).view(np.int16)).view(torch.bfloat16).clone()
    y_host = torch.full((tokens, h), float("nan"), dtype=torch.bfloat16)
    if pinned:
        x_host, y_host = x_host.pin_memory(), y_host.pin_memory()
    staging = torch.empty((2 * tokens, h), dtype=torch.bfloat16, device=cuda)
    ws = mlp.workspace(tokens)
    for _ in range(3):
        y_host.fill_(float("nan"))
        forward_mlp_host(mlp, x_host, y_host, staging, ws)      # no synchronize here: the call is synchronous
        got = y_host.float().numpy().copy()
        assert_ffn_close(got, want, f"host entry, {'pinned' if pinned else 'pageable'}, M={tokens}")
    call = bind_forward_mlp_host(mlp, x_host, y_host, staging, ws)   # the same call with its arguments converted once
    y_host.fill_(float("nan"))
    call()
    assert np.array_equal(y_host.view(torch.int16).numpy(), o.bf16_bits(got).view(np.int16))
    L.device_status()
