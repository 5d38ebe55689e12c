"""The batched FFN (3..64 tokens per pass) on the tcgen05 tensor cores against the CPU oracle, next to
the mma.sync pair it replaces by default (ffn_int4_set_batched_kernel): same bars, same workspace
contract, repeatable bit for bit."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import ffn_oracle as o
from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer
from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200.ops import decode_stack

pytestmark = pytest.mark.gpu

KERNELS = {"tcgen05": 0, "mma.sync": 1}


@pytest.fixture(params=list(KERNELS), autouse=True)
def batched_kernel(request):
    old = L.load().ffn_int4_set_batched_kernel(KERNELS[request.param])
    yield request.param
    L.load().ffn_int4_set_batched_kernel(old)


@pytest.fixture(scope="module")
def drawn():
    cache = {}

    def get(cfg, tokens):
        if (cfg, tokens) not in cache:
            if len(cache) > 3:
                cache.clear()
            spec = o.CONFIGS[cfg]
            x, layers = o.draw_config(spec["hidden"], spec["inter"], spec["seed"], tokens=tokens)
            want, _, act = None, None, None
            want, _, act = o.ffn(layers[0], x, intermediates=True)
            cache[(cfg, tokens)] = (x, layers[0], want, act)
        return cache[(cfg, tokens)]
    return get


def plan_text(tokens, hidden, inter):
    buf = ctypes.create_string_buffer(1024)
    L.check(L.load().ffn_int4_describe_plan(tokens, hidden, inter, 148, 232448, buf, len(buf)))
    return buf.value.decode()


@pytest.mark.parametrize("cfg,tokens", [(0, 3), (0, 8), (0, 16), (0, 17), (0, 33), (0, 48), (0, 64), (0, 100),
                                        (1, 5), (1, 64), (2, 16), (2, 64)])
def test_batched_pair_matches_oracle(cuda, drawn, batched_kernel, cfg, tokens):
    spec = o.CONFIGS[cfg]
    x, layer, want, act = drawn(cfg, tokens)
    expect = "kernel=tcgen05_pair" if batched_kernel == "tcgen05" else "kernel=mma_pair"
    assert expect in plan_text(tokens, spec["hidden"], spec["inter"])
    mlp = upload_layer(layer, cuda)
    ws = mlp.workspace(tokens)
    xd = dev_bf16(x, cuda)
    got_t = mlp.forward_mlp_prepared(xd, ws=ws)
    L.device_status()
    max_abs, rel = assert_ffn_close(host_f32(got_t), want, f"{batched_kernel} config {cfg} M={tokens}")
    print(f"{batched_kernel} config {cfg} M={tokens}: max-abs {max_abs:.3g} rel-L2 {rel:.3g}")
    h, i = spec["hidden"], spec["inter"]
    got_act = host_f32(ws[tokens * (h + 2 * i):tokens * (h + 3 * i)].view(tokens, i))
    assert o.compare(got_act, act)[1] <= 5e-3            # act is left in the caller's workspace, natural order
    for _ in range(3):                                   # fixed summation order: repeatable bit for bit
        again = mlp.forward_mlp_prepared(xd, ws=ws)
        assert torch.equal(again.view(torch.int16), got_t.view(torch.int16))
    L.device_status()


@pytest.mark.parametrize("tokens", [8, 40])
def test_batched_pair_in_a_stack_with_norm_and_residual(cuda, batched_kernel, tokens):
    """h <- h + FFN(RMSNorm(h)) through three layers: the down launch's fused residual update."""
    hidden, inter = 1024, 3072
    h0, layers = o.draw_config(hidden, inter, 11, tokens=tokens, layers=3, with_norm=True)
    ref = o.stack(layers, h0)
    mlps = [upload_layer(lay, cuda, with_norm=True) for lay in layers]
    inputs = [h0] + ref[:-1]
    for l, mlp in enumerate(mlps):
        h = dev_bf16(inputs[l], cuda).clone()
        decode_stack([mlp], h)
        L.device_status()
        assert_ffn_close(host_f32(h), ref[l], f"{batched_kernel} layer {l} teacher-forced, M={tokens}")


def test_token_counts_alternate_on_one_device(cuda, drawn):
    """Different token paddings one after the other: stale columns of the tile-order scratch (tokens
    beyond the current count) never reach an output."""
    for cfg, tokens in [(0, 64), (0, 3), (0, 33), (0, 16), (0, 64), (0, 17)]:
        x, layer, want, _ = drawn(cfg, tokens)
        mlp = upload_layer(layer, cuda)
        got = host_f32(mlp.forward_mlp_prepared(dev_bf16(x, cuda)))
        L.device_status()
        assert_ffn_close(got, want, f"config {cfg} M={tokens} in a mixed sequence")


def test_non_finite_input_stays_in_its_token(cuda, drawn):
    """A NaN in one token's input poisons that token's outputs only (columns of the MMA are independent)."""
    x, layer, want, _ = drawn(0, 16)
    xp = x.copy()
    xp[5, 100] = np.nan
    mlp = upload_layer(layer, cuda)
    got = host_f32(mlp.forward_mlp_prepared(dev_bf16(xp, cuda)))
    L.device_status()
    assert np.isnan(got[5]).all()
    keep = [m for m in range(16) if m != 5]
    assert_ffn_close(got[keep], want[keep], "the other tokens")
