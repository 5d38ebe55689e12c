"""Pipeline timelines of the decode and batched kernels from their own clock stamps (ffn_int4_debug_trace).

    python -m haskell_infer_demo_b200.trace decode  [--hidden H] [--inter I] [--tokens M] [--kmajor] [--graph]
    python -m haskell_infer_demo_b200.trace batched [--hidden H] [--inter I] [--tokens M]

`decode`: every CTA of a one- or two-token launch stamps the global timer at its pipeline events; the
table gives min / median / max over the CTAs in microseconds after the first CTA's start.  --kmajor
registers the k-major copy first (the persistent kernel of ffn_decode_layer_prepare); --graph takes the
stamps of the last of twelve back-to-back launches in a CUDA graph instead of a launch on an idle device.
`batched`: CTA 0 of the tcgen05 pair stamps the SM clock per role and 128-wide group (gate/up launch and
down launch).  Weights are random codes with a constant scale: the timing does not depend on the values.
Needs a B200; a measuring aid, not part of the drop-in.
"""
import argparse
import ctypes

import numpy as np
import torch

from . import lib as L
from .ops import DenseMlp

ROW_MAJOR = {0: "start", 1: "producer past the dependency wait", 2: "input prepared", 3: "phase 1 first tile",
             4: "phase 1 consumers done", 5: "grid barrier arrival", 6: "grid barrier open", 7: "act prepared",
             8: "phase 2 first tile", 9: "phase 2 consumers done", 10: "epilogue done", 11: "peer sums added", 12: "exit"}
K_MAJOR = {0: "start", 1: "producer go", 2: "input prepared", 3: "phase 1 first tile", 4: "phase 1 consumers done",
           5: "act ready", 6: "consumers past act ready", 7: "phase 2 first tile", 8: "partials stored",
           13: "arrival counter seen", 10: "reducers released", 11: "partials read", 9: "reduced and written", 12: "exit"}
TC_ROLES = ["stage issued", "conversion start", "conversion done", "MMA issue start", "MMAs committed", "epilogue got group",
            "epilogue done"]


def random_layer(hidden, inter, dev):
    gu = torch.randint(0, 256, (2 * inter, hidden // 2), dtype=torch.uint8, device=dev) & 0x77
    gus = torch.full((2 * inter, hidden // 128), 0.01, dtype=torch.bfloat16, device=dev)
    dn = torch.randint(0, 256, (hidden, inter // 2), dtype=torch.uint8, device=dev) & 0x77
    dns = torch.full((hidden, inter // 128), 0.01, dtype=torch.bfloat16, device=dev)
    return DenseMlp(gu, gus, dn, dns)


def stamped_call(calls, graph):
    """Runs `calls` (a list of zero-argument launches, used round robin) warm, then once more - or as the
    last of twelve in a graph - with the trace buffer registered; returns the buffer as int64 numpy."""
    lib = L.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    buf = torch.zeros(max(16 * sms, 1024), dtype=torch.int64, device=dev)
    for k in range(3):
        calls[k % len(calls)]()
    torch.cuda.synchronize()
    lib.ffn_int4_debug_trace(ctypes.c_void_p(buf.data_ptr()))
    try:
        if graph:
            stream, g = torch.cuda.Stream(), torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(g, stream=stream):
                    for k in range(12):
                        calls[k % len(calls)]()
                g.replay()
        else:
            calls[0]()
        torch.cuda.synchronize()
        L.device_status()
    finally:
        lib.ffn_int4_debug_trace(None)
    return buf.cpu().numpy(), sms


def decode(args):
    dev = torch.device("cuda", 0)
    copies = 4 if args.graph else 1
    mlps = [random_layer(args.hidden, args.inter, dev) for _ in range(copies)]
    if args.kmajor:
        for mlp in mlps:
            mlp.prepare()
    x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
    ws = mlps[0].workspace(args.tokens)
    out = torch.empty_like(x)
    raw, sms = stamped_call([lambda mlp=mlp: mlp.forward_mlp_prepared(x, ws=ws, layer_out=out) for mlp in mlps], args.graph)
    t = raw[:16 * sms].reshape(sms, 16).astype(np.float64)
    t0 = t[:, 0][t[:, 0] > 0].min()
    names = K_MAJOR if args.kmajor else ROW_MAJOR
    print(f"{'k-major' if args.kmajor else 'row-major'} decode kernel, H={args.hidden} I={args.inter} M={args.tokens}"
          f"{', last of 12 launches in a graph' if args.graph else ''}: us after the first CTA's start, min / median / max over CTAs")
    for slot, name in names.items():
        col = t[:, slot]
        col = col[col > 0]
        if len(col):
            print(f"  {name:36s} {(col.min() - t0) / 1e3:8.2f} {(np.median(col) - t0) / 1e3:8.2f} {(col.max() - t0) / 1e3:8.2f}   ({len(col)} CTAs)")


def batched(args):
    lib = L.load()
    dev = torch.device("cuda", 0)
    mlp = random_layer(args.hidden, args.inter, dev)
    x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
    ws = mlp.workspace(args.tokens)
    out = torch.empty_like(x)
    old = lib.ffn_int4_set_batched_kernel(0)
    try:
        raw, _ = stamped_call([lambda: mlp.forward_mlp_prepared(x, ws=ws, layer_out=out)], False)
    finally:
        lib.ffn_int4_set_batched_kernel(old)
    for which, base in (("gate/up", 0), ("down", 512)):
        t = raw[base:base + 8 * 64].reshape(8, 64).astype(np.float64)
        if not (t > 0).any():
            print(f"{which} launch: no stamps (the shape went to the mma.sync pair)")
            continue
        t0 = t[t > 0].min()
        print(f"tcgen05 pair, {which} launch, H={args.hidden} I={args.inter} M={args.tokens}: CTA 0, SM clock cycles after its first stamp")
        ev = t[7, :3]
        print("  epilogue: first unit starts %.0f, its group loop ends %.0f, its output is written %.0f" % tuple(np.where(ev > 0, ev - t0, -1)))
        print("  group " + " ".join(f"{n:>18s}" for n in TC_ROLES))
        for g in range(0, 64, args.every):
            if (t[:7, g] > 0).any():
                print(f"  {g:5d} " + " ".join(f"{t[r, g] - t0:18.0f}" if t[r, g] > 0 else " " * 18 for r in range(7)))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["decode", "batched"])
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--inter", type=int, default=17408)
    ap.add_argument("--tokens", type=int, default=0, help="default: 1 for decode, 64 for batched")
    ap.add_argument("--kmajor", action="store_true")
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--every", type=int, default=4, help="batched: print every n-th group")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the timelines come from a B200; no CUDA device here")
    if args.tokens == 0:
        args.tokens = 1 if args.what == "decode" else 64
    (decode if args.what == "decode" else batched)(args)


if __name__ == "__main__":
    main()
