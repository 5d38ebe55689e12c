"""GPU parity of the decode kernel over k-major copies of the down projection (ffn_decode_layer_prepare):
the same entry points and the same bars as the row-major kernel, plus what is particular to it - CTAs
without any K range, a K range that straddles scale groups, the residual stream handed from layer to
layer inside one launch, launches of both kernels alternating on one device."""
import ctypes

import numpy as np
import pytest
import torch

from haskell_infer_demo_b200 import lib as L
from haskell_infer_demo_b200.ops import decode_stack
from oracle import ffn_oracle as o
from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer

pytestmark = pytest.mark.gpu

SHAPES = [(1024, 3072, 0), (2560, 9728, 1), (5120, 17408, 2),
          (1024, 384, 5),      # fewer k-blocks (48) than CTAs: most CTAs own no K range at all
          (5120, 2176, 6),     # the 27B layer's slice at TP=8: one or two k-blocks per CTA
          (128, 128, 7),       # fewer output rows than CTAs
          (2560, 4864, 8), (6528, 1024, 9)]   # the widest hidden size the kernel takes


@pytest.fixture(params=[0, 1], ids=["tensor-core", "dp4a"], autouse=True)
def decode_kernel(request):
    """Every test of this file runs twice: with the dp4a kernel, which is the default for prepared
    layers, and with the opt-in tensor-core (INT8 MMA) consumers (ffn_int4_set_decode_kernel)."""
    old = L.load().ffn_int4_set_decode_kernel(request.param)
    yield request.param
    L.load().ffn_int4_set_decode_kernel(old)


@pytest.fixture(scope="module")
def drawn():
    cache = {}

    def get(h, i, seed, tokens):
        if (h, i, seed, tokens) not in cache:
            if len(cache) > 4:
                cache.clear()
            x, layers = o.draw_config(h, i, seed, tokens=tokens)
            cache[(h, i, seed, tokens)] = (x, layers[0], o.ffn(layers[0], x))
        return cache[(h, i, seed, tokens)]
    return get


@pytest.mark.parametrize("tokens", [1, 2, 3, 4])
@pytest.mark.parametrize("hidden,inter,seed", SHAPES)
def test_kmajor_ffn_matches_oracle(cuda, drawn, decode_kernel, hidden, inter, seed, tokens):
    if tokens > 2 and decode_kernel == 1:
        pytest.skip("the dp4a kernel takes one or two tokens")
    x, layer, want = drawn(hidden, inter, seed, tokens)
    mlp = upload_layer(layer, cuda, prepare=True)
    assert L.load().ffn_decode_layer_is_prepared(ctypes.byref(mlp.weights)) == 1
    plan = ctypes.create_string_buffer(1024)
    L.check(L.load().ffn_int4_describe_kmajor_plan(tokens, hidden, inter, 148, 232448, plan, 1024))
    if tokens <= 2:      # (three and four tokens fall back to the batched pair where the tensor-core kernel has no room)
        assert b"kernel=imma" in plan.value or b"kernel=kmajor" in plan.value, plan.value
    xd = dev_bf16(x, cuda)
    ws = mlp.workspace(tokens)
    got_t = mlp.forward_mlp_prepared(xd, ws=ws)
    L.device_status()
    assert_ffn_close(host_f32(got_t), want, f"k-major H={hidden} I={inter} M={tokens}")
    # the activation is left in the caller's workspace as the reference leaves it
    _, _, act = o.ffn(layer, x, intermediates=True)
    got_act = host_f32(ws[tokens * (hidden + 2 * inter):tokens * (hidden + 3 * inter)].view(tokens, inter))
    assert o.compare(got_act, act)[1] <= 5e-3
    # repeatable bit for bit (fixed summation order, self-validating hand-over words)
    for _ in range(10):
        again = mlp.forward_mlp_prepared(xd, ws=ws)
        assert torch.equal(again.view(torch.int16), got_t.view(torch.int16))
    L.device_status()
    # and really another kernel than the row-major one: releasing the copy changes the route, not the answer
    mlp.release()
    assert L.load().ffn_decode_layer_is_prepared(ctypes.byref(mlp.weights)) == 0
    row_major = mlp.forward_mlp_prepared(xd, ws=ws)
    L.device_status()
    assert_ffn_close(host_f32(row_major), want, "row-major after release")


def test_kernels_alternate_on_one_device(cuda, drawn):
    """Row-major and k-major launches, different shapes and token counts, one after the other: neither
    kernel may see the other's (or its own earlier launch's) hand-over words as current."""
    order = [(1024, 3072, 0, 1, True), (2560, 9728, 1, 2, False), (1024, 3072, 0, 2, True), (1024, 384, 5, 1, True),
             (2560, 9728, 1, 1, True), (1024, 3072, 0, 1, False), (2560, 9728, 1, 2, True), (1024, 384, 5, 2, True)]
    mlps = {}
    for h, i, seed, tokens, prep in order:
        x, layer, want = drawn(h, i, seed, tokens)
        key = (h, i, seed, tokens, prep)
        if key not in mlps:
            mlps[key] = upload_layer(layer, cuda, prepare=prep)
        got = host_f32(mlps[key].forward_mlp_prepared(dev_bf16(x, cuda)))
        L.device_status()
        assert_ffn_close(got, want, f"H={h} I={i} M={tokens} prepared={prep} in a mixed sequence")


@pytest.mark.parametrize("tokens,nlayers", [(1, 12), (2, 7), (4, 5)])
def test_kmajor_stack_one_launch(cuda, decode_kernel, tokens, nlayers):
    if tokens > 2 and decode_kernel == 1:
        pytest.skip("the dp4a kernel takes one or two tokens")
    """The stack in ONE persistent launch: teacher-forced per layer at the FFN bars, free-running
    within the oracle-vs-oracle spread, equal bit for bit to the same layers launched one by one, and
    to itself when run again."""
    hidden, inter = 1024, 3072
    h0, layers = o.draw_config(hidden, inter, 4, tokens=tokens, layers=nlayers, with_norm=True)
    ref64 = o.stack(layers, h0)
    ref32 = o.stack(layers, h0, accumulate="f32")
    mlps = [upload_layer(lay, cuda, with_norm=True, prepare=True) for lay in layers]
    inputs = [h0] + ref64[:-1]
    for l in range(nlayers):
        h = dev_bf16(inputs[l], cuda).clone()
        decode_stack([mlps[l]], h)
        L.device_status()
        assert_ffn_close(host_f32(h), ref64[l], f"k-major layer {l} teacher-forced, M={tokens}")
    h = dev_bf16(h0, cuda).clone()
    y = torch.empty_like(h)
    decode_stack(mlps, h, layer_out=y)
    L.device_status()
    _, spread = o.compare(ref32[-1], ref64[-1])
    _, rel = o.compare(host_f32(h), ref64[-1])
    print(f"k-major M={tokens} L={nlayers}: free-running rel-L2 {rel:.3g}; oracle-vs-oracle spread {spread:.3g}")
    assert rel <= max(5e-3, 2 * spread)
    h2 = dev_bf16(h0, cuda).clone()
    y2 = torch.empty_like(h2)
    for m in mlps:
        decode_stack([m], h2, layer_out=y2)
    L.device_status()
    assert torch.equal(h2.view(torch.int16), h.view(torch.int16))
    assert torch.equal(y2.view(torch.int16), y.view(torch.int16))      # layer_out holds the last layer's FFN output
    h3 = dev_bf16(h0, cuda).clone()
    decode_stack(mlps, h3)
    L.device_status()
    assert torch.equal(h3.view(torch.int16), h.view(torch.int16))


def test_kmajor_more_layers_than_one_launch_takes(cuda):
    """70 layers = one launch of 64 and one of 6 (the layers' pointers travel in the kernel parameters)."""
    hidden, inter, nlayers = 256, 512, 70
    h0, layers = o.draw_config(hidden, inter, 11, layers=nlayers, with_norm=True)
    ref = o.stack(layers, h0)
    mlps = [upload_layer(lay, cuda, with_norm=True, prepare=True) for lay in layers]
    h = dev_bf16(h0, cuda).clone()
    decode_stack(mlps, h)
    L.device_status()
    h2 = dev_bf16(h0, cuda).clone()
    for m in mlps:
        decode_stack([m], h2)
    L.device_status()
    assert torch.equal(h2.view(torch.int16), h.view(torch.int16))
    # 70 free-running layers of a narrow model are chaotic under BF16 rounding (one rounding that falls
    # differently decorrelates the stream), so this is a sanity bound; the per-layer bars are held by the
    # teacher-forced tests, and the launches' equality with the layer-by-layer run is exact above
    assert o.compare(host_f32(h), ref[-1])[1] <= 3e-2
    for l in (0, 63, 64, 69):                                 # either side of the launch boundary
        hl = dev_bf16(h0 if l == 0 else ref[l - 1], cuda).clone()
        decode_stack([mlps[l]], hl)
        L.device_status()
        assert_ffn_close(host_f32(hl), ref[l], f"layer {l} of 70 teacher-forced")


def test_kmajor_residual_and_norm_variants(cuda):
    """forward_mlp (separate norm kernel, no residual) and the fused residual update of the TP entry at
    one rank both reach the k-major kernel; a non-finite activation still poisons its token's outputs."""
    from haskell_infer_demo_b200.ops import TpComm
    hidden, inter = 1024, 3072
    x, layers = o.draw_config(hidden, inter, 7, tokens=2, with_norm=True)
    lay = layers[0]
    mlp = upload_layer(lay, cuda, with_norm=True, prepare=True)
    got = host_f32(mlp.forward_mlp(dev_bf16(x, cuda)))
    L.device_status()
    assert o.compare(got, o.ffn(lay, o.gemma_rmsnorm(x, lay.w_norm)))[1] <= 5e-3
    comm = TpComm.local([cuda], hidden, 2)[0]
    try:
        hres = o.bf16_round(np.random.default_rng(5).standard_normal((2, hidden), dtype=np.float32))
        res = dev_bf16(hres, cuda).clone()
        y = comm.forward_mlp(mlp, dev_bf16(x, cuda), residual=res)
        L.device_status()
        assert_ffn_close(host_f32(y), o.ffn(lay, x), "k-major with a separate residual buffer")
        assert np.array_equal(host_f32(res), o.residual_add(hres, host_f32(y)))
    finally:
        comm.close()
    xd = dev_bf16(x, cuda).clone()
    xd[1, 77] = float("nan")
    y = host_f32(mlp.forward_mlp_prepared(xd))
    L.device_status()
    assert not np.isfinite(y[1]).any() and np.isfinite(y[0]).all()
