"""Generates tests/golden/stack_cfg4.npz: the CPU oracle's trajectory through the 64-layer stack of
27B-shape INT4 FFNs (BASELINE configs[4]: h <- h + FFN_l(GemmaRMSNorm_l(h)), identity mixers).

    python tests/golden/make_stack_golden.py [--layers 64] [--out tests/golden/stack_cfg4.npz]

The 17 G weights are the counter-based synthetic ones of haskell_infer_demo_b200.synth (seed 4): a
pure function of (seed, tensor, layer, element index), so the GPU tests regenerate any rank's slice
on the device in seconds while this script, run once on a CPU box, supplies the expected states.
Quantization and the FFN chain are the oracle's (oracle/ffn_oracle.py).  Tokens are independent, so
one pass with eight tokens serves the one-token case too (token 0).

Stored (BF16 bit patterns):
  tok0_states [L][H]        h after every layer, token 0 (teacher forcing of all layers at M=1)
  tok0_ffn_out [L][H]       the FFN output y_l of every layer, token 0: the residual stream grows to
                            |h| ~ 100 over 64 layers (one BF16 ulp of h then exceeds the whole error
                            budget of y), so the per-layer gate compares y, and checks h = bf16(h + y)
                            exactly
  m8_layers   [n]           the layers whose input and output states are kept for all eight tokens
  m8_states   [n][2][8][H]  h before and after those layers, tokens 0..7
  m8_ffn_out  [n][8][H]     their FFN outputs
  final_f64 / final_f32 [8][H]  free-running final state with FP64- / FP32-accumulating matmuls
  spread_rel_l2             relative L2 between the two finals: the oracle-vs-oracle spread that
                            bounds what any implementation with other summation orders can match
  digest_layer0             SHA-256 of layer 0's gate||up packed bytes, scales, down packed bytes,
                            down scales (the device-side generator + quantizer must reproduce them)
"""
import argparse
import hashlib
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from haskell_infer_demo_b200 import synth  # noqa: E402
from oracle import ffn_oracle as o  # noqa: E402

SEED, HIDDEN, INTER, TOKENS = 4, 5120, 17408, 8
M8_LAYERS = [0, 1, 31, 62, 63]


def draw_layer(layer, hidden, inter):
    gp, gs = o.quantize(synth.matrix_numpy(SEED, synth.W_GATE, layer, inter, hidden, 0.02))
    up, us = o.quantize(synth.matrix_numpy(SEED, synth.W_UP, layer, inter, hidden, 0.02))
    dp, ds = o.quantize(synth.matrix_numpy(SEED, synth.W_DOWN, layer, hidden, inter, 0.02))
    w_norm = o.bf16_round(synth.matrix_numpy(SEED, synth.W_NORM, layer, 1, hidden, 0.1).reshape(hidden))
    return o.Layer(np.concatenate([gp, up]), np.concatenate([gs, us]), dp, ds, w_norm)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=HIDDEN)
    ap.add_argument("--inter", type=int, default=INTER)
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "stack_cfg4.npz"))
    args = ap.parse_args()
    nl, hidden, inter = args.layers, args.hidden, args.inter
    keep = [l for l in M8_LAYERS if l < nl]
    h64 = o.bf16_round(synth.matrix_numpy(SEED, synth.X, 0, TOKENS, hidden, 1.0))
    h32 = h64.copy()
    tok0 = np.zeros((nl, hidden), np.uint16)
    m8 = np.zeros((len(keep), 2, TOKENS, hidden), np.uint16)
    tok0_y = np.zeros((nl, hidden), np.uint16)
    m8_y = np.zeros((len(keep), TOKENS, hidden), np.uint16)
    digest = ""
    t0 = time.time()
    for l in range(nl):
        lay = draw_layer(l, hidden, inter)
        if l == 0:
            digest = ",".join(hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
                              for a in (lay.gate_up_packed, lay.gate_up_scales, lay.down_packed, lay.down_scales))
        if l in keep:
            m8[keep.index(l), 0] = o.bf16_bits(h64)
        y64 = o.ffn(lay, o.gemma_rmsnorm(h64, lay.w_norm))
        h64 = o.residual_add(h64, y64)
        h32 = o.stack([lay], h32, accumulate="f32")[0]
        tok0[l] = o.bf16_bits(h64[0])
        tok0_y[l] = o.bf16_bits(y64[0])
        if l in keep:
            m8[keep.index(l), 1] = o.bf16_bits(h64)
            m8_y[keep.index(l)] = o.bf16_bits(y64)
        print(f"layer {l}: {time.time() - t0:.0f} s, |h| rms {np.sqrt((h64 ** 2).mean()):.3f}, "
              f"f32-vs-f64 rel-L2 so far {o.compare(h32, h64)[1]:.3g}", flush=True)
    spread = o.compare(h32, h64)[1]
    spread0 = o.compare(h32[:1], h64[:1])[1]
    np.savez_compressed(args.out, tok0_states=tok0, tok0_ffn_out=tok0_y, m8_layers=np.array(keep), m8_states=m8, m8_ffn_out=m8_y,
                        final_f64=o.bf16_bits(h64), final_f32=o.bf16_bits(h32), spread_rel_l2=np.float64(spread),
                        spread_rel_l2_token0=np.float64(spread0), digest_layer0=np.array(digest),
                        shape=np.array([nl, hidden, inter, TOKENS, SEED]))
    print(f"wrote {args.out}: spread {spread:.3g} (token 0: {spread0:.3g})")


if __name__ == "__main__":
    main()
