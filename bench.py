"""Benchmark of the INT4 dense-FFN decode path (metric of BASELINE.json: µs/step and HBM GB/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens M]

N = 1   one 27B-shape FFN (H=5120, I=17408, M=1, TP=1; BASELINE.json configs[2]) per step.
N > 1   launched by torchrun, one rank per GPU: the same layer under tensor parallelism TP=N, every
        rank reading only its slice, the down projection's partial sums reduced inside the kernel
        over NVLink (strong scaling: the total work is fixed).

A step is one FFN call through the C ABI (ffn_forward_mlp_prepared / ffn_forward_mlp_tp).  Steps
rotate through enough distinct weight copies that the bytes touched between two uses of one copy
exceed twice the L2 (so "HBM GB/s" is an HBM number).  `value` is device time per step with inputs
resident in HBM (K steps captured in one CUDA graph, CUDA events on the launching stream, max over
ranks); `e2e` is the same call fed from pinned HOST buffers with the H2D copy of x and the D2H copy
of y inside the timed region.  `roofline` uses the algorithmic bytes per step per rank
(packed weights + BF16 scales = 1.546875*H*I/TP) against the measured copy peak.  `cpu_baseline`
times the CPU oracle chain on this box's host cores on a bounded sample.

--impl reference times the reference's own CPU arithmetic for the path on the host cores (the
reference's compiled dequantizer from oracle/_ref when present, else the oracle's restatement;
matmuls in PyTorch on all host threads) and prints the same JSON line with "impl": "reference".
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER = 5120, 17408
L2_BYTES = 126 * 1024 * 1024
METRIC = "int4_ffn_decode_us_per_step"
# dram__bytes_read.sum + dram__bytes_write.sum of one fused launch at H=5120, I=17408, M=1, TP=1 (ncu --set
# full capture summarised in profiles/ffn_fused_kernel_cfg2_tp1.md); other shapes have no capture yet.
TRAFFIC_BYTES = {(1, 1): 144.94e6}


def algorithmic_bytes(h, i, tp):
    return 1.546875 * h * i / tp


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def stop(self):
        if self.proc:
            self.proc.terminate()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(s[2 + k].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in self.samples),
                "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons, "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# synthetic layer, generated on the device (N(0, 0.02) weights quantized with the format's rule)
# ------------------------------------------------------------------------------------------------
def quantize_on_device(w):
    """The library's GPU quantizer (byte-identical to the reference's format)."""
    from haskell_infer_demo_b200.ops import quantize_int4
    return quantize_int4(w.contiguous())


def make_rank_layer(dev, h, i, tp, rank, seed):
    """This rank's slice of one layer: gate/up rows and down columns [rank*I/tp, (rank+1)*I/tp)."""
    import torch
    from haskell_infer_demo_b200.ops import DenseMlp
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    per = i // tp
    parts = []
    for _ in range(2):  # gate, up: draw the whole tensor row block by row block, keep this rank's rows
        w = torch.randn((per, h), generator=gen, device=dev) * 0.02
        parts.append(quantize_on_device(w))
    gu_p = torch.cat([parts[0][0], parts[1][0]])
    gu_s = torch.cat([parts[0][1], parts[1][1]])
    wd = torch.randn((h, per), generator=gen, device=dev) * 0.02
    d_p, d_s = quantize_on_device(wd)
    return DenseMlp(gu_p, gu_s, d_p, d_s)


def clone_layer(mlp):
    from haskell_infer_demo_b200.ops import DenseMlp
    t = mlp.tensors
    return DenseMlp(t[0].clone(), t[1].clone(), t[2].clone(), t[3].clone())


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import TpComm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = L.load()
    tp, m, h, i = world, args.tokens, HIDDEN, INTER
    per_rank_bytes = algorithmic_bytes(h, i, tp)
    copies = max(2, int(2.2 * L2_BYTES / per_rank_bytes) + 1)
    if args.layers > 0:
        copies = args.layers
    base = make_rank_layer(dev, h, i, tp, rank, seed=2)
    layers = [base] + [clone_layer(base) for _ in range(copies - 1)]
    if args.layers > 0:  # every layer gets a Gemma norm weight ~ N(0, 0.1)
        import torch as _t
        from haskell_infer_demo_b200.ops import DenseMlp, decode_stack
        g = _t.Generator(device=dev)
        g.manual_seed(99)
        layers = [DenseMlp(*lay.tensors[:4], post_norm_w=(_t.randn(h, generator=g, device=dev) * 0.1).to(_t.bfloat16))
                  for lay in layers]
    use_nccl = world > 1 and args.exchange == "nccl"
    if use_nccl and args.layers > 0:
        raise SystemExit("--exchange nccl is a single-layer comparison; drop --layers")
    comm = TpComm.over_process_group(h, max(m, 2)) if world > 1 and not use_nccl else None
    nl = max(args.layers, 1)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    x = torch.randn((m, h), generator=gen, device=dev).to(torch.bfloat16)
    ws = base.workspace(m)
    out = torch.empty((m, h), dtype=torch.bfloat16, device=dev)

    hstate = x.clone()

    def step(k):
        if args.layers > 0:
            hstate.copy_(x)  # restart the residual stream so its magnitude does not drift over the run
            decode_stack(layers, hstate, comm=comm, ws=ws, layer_out=out)
            return
        lay = layers[k % copies]
        if comm is None:
            lay.forward_mlp_prepared(x, ws=ws, layer_out=out)
            if use_nccl:
                dist.all_reduce(out)
        else:
            comm.forward_mlp(lay, x, ws=ws, layer_out=out)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for k in range(max(args.warmup, 3)):
        step(k)
    barrier()
    L.device_status()

    # ---- device-resident timing: K steps in one graph, events on the launching stream
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for k in range(args.steps):
                step(k)
        graph.replay()  # untimed: first replay uploads the graph
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # One more untimed replay tells how many timed replays make the region long enough (about 0.6 s) for the
    # clock sampler to see it several times; every rank must agree on the count.
    with torch.cuda.stream(stream):
        e0.record(stream)
        graph.replay()
        e1.record(stream)
    barrier()
    est = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    reps, times = int(min(400, max(5, -(-600.0 // max(float(est.item()), 1e-3))))), []
    for _ in range(reps):
        barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        barrier()
        times.append(e0.elapsed_time(e1))
    ms_total = statistics.median(times)
    L.device_status()

    # ---- end to end: host buffers in, host buffer out, every step
    x_host = x.cpu().pin_memory()
    y_host = torch.empty((m, h), dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty_like(x)
    e2e_steps = args.steps
    cur = torch.cuda.current_stream()

    def e2e_step(k):
        x_dev.copy_(x_host, non_blocking=True)
        lay = layers[k % copies]
        if args.layers > 0:
            decode_stack(layers, x_dev, comm=comm, ws=ws, layer_out=out)
            y_host.copy_(x_dev, non_blocking=True)
        elif comm is None:
            lay.forward_mlp_prepared(x_dev, ws=ws, layer_out=out)
            if use_nccl:
                dist.all_reduce(out)
            y_host.copy_(out, non_blocking=True)
        else:
            comm.forward_mlp(lay, x_dev, ws=ws, layer_out=out)
            y_host.copy_(out, non_blocking=True)
        cur.synchronize()  # the caller needs this step's result before it can issue the next one

    for k in range(3):
        e2e_step(k)
    barrier()
    e0.record()
    for k in range(e2e_steps):
        e2e_step(k)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms_total, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = t.tolist()
    us_step = ms_total * 1e3 / args.steps
    e2e_us = e2e_ms * 1e3 / e2e_steps
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        gbs = nl * per_rank_bytes / us_step / 1e3
        line = {
            "metric": METRIC, "value": round(us_step, 3), "unit": "us/step", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(us_step / 1e3, 6),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "int4xbf16->f32",
            "data": "synthetic (N(0,0.02) weights quantized on the device, N(0,1) BF16 activations)",
            "tokens_per_s": round(m * 1e6 / us_step, 1),
            "hbm_gbs_per_gpu": round(gbs, 1), "pct_of_8tbs": round(gbs / 80.0, 2),
            "config": {"workload": (f"27B-shape INT4 FFN decode H={h} I={i} M={m} TP={tp} (BASELINE configs[2])" if not args.layers else
                                    f"{args.layers}-layer stack h+=FFN(GemmaRMSNorm(h)), H={h} I={i} M={m} TP={tp} (BASELINE configs[4])"),
                       "l2": f"rotating {copies} weight copies per rank ({copies * per_rank_bytes / 1e6:.0f} MB > 2x L2)",
                       "timing": f"{args.steps} steps in one CUDA graph, median of {reps} replays, max over ranks"},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(gbs / peak, 4), "peak_source": peak_kind, "traffic": TRAFFIC_BYTES.get((tp, m)) if not args.layers else None,
                         "algorithmic_bytes_per_launch": per_rank_bytes, "launches_per_step": nl},
            "e2e": {"value": round(e2e_us, 3), "unit": "us/step", "h2d_bytes_per_step": m * h * 2,
                    "d2h_bytes_per_step": m * h * 2},
            "gpu_launches": args.steps * nl * (1 if m <= 2 else (4 if args.layers else 3)),
            "exchange": ("none (one GPU)" if world == 1 else "in-kernel tagged-word exchange over NVLink peer memory"
                         if not use_nccl else "comparison variant: NCCL all-reduce of the BF16 output after the kernel"),
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu and not args.layers:
            line["cpu_baseline"] = cpu_baseline(h, i, m, budget_s=12.0)
        print(json.dumps(line), flush=True)
    if comm is not None:
        barrier()
        comm.close()
        dist.destroy_process_group()
    # The comparison variant leaves its process group to interpreter exit: tearing NCCL down while the
    # captured graph that holds its collectives is alive did not return on 8 GPUs.


# ------------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------------
def cpu_baseline(h, i, m, budget_s):
    """The oracle chain (FP64-accumulating C loops over the packed bytes, one thread) on a bounded
    sample: whole steps of the same workload until the budget is spent."""
    import numpy as np
    from oracle import ffn_oracle as o
    x, layers = o.draw_config(h, i, 2, tokens=m)
    lay = layers[0]
    o.ffn(lay, x)
    t0, n = time.perf_counter(), 0
    while n < 2 or (time.perf_counter() - t0 < budget_s and n < 50):
        o.ffn(lay, x)
        n += 1
    us = (time.perf_counter() - t0) / n * 1e6
    return {"value": round(us, 1), "unit": "us/step", "cores": 1, "kind": "port",
            "sample": f"{n} whole steps of the same layer (oracle chain from packed bytes, FP64 accumulation)"}


def run_reference(args):
    """The reference's CPU arithmetic for the path, all host threads: dequantize with the
    reference's own linear_dequantize_int4 when oracle/_ref holds it, FP32 matmuls in PyTorch with
    the reference's three BF16 rounding points."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ctypes
    import numpy as np
    import torch
    from oracle import ffn_oracle as o
    h, i, m = HIDDEN, INTER, args.tokens
    x, layers = o.draw_config(h, i, 2, tokens=m)
    lay = layers[0]
    ref = o.ref_lib()
    kind = "reference" if ref is not None else "port"

    class Layout(ctypes.Structure):
        _fields_ = [(n, ctypes.c_longlong) for n in ("n", "k", "group", "packed_bytes", "scale_count")]

    def dequant(packed, scales):
        if ref is None:
            return o.dequantize(packed, scales)
        n, kb = packed.shape
        lo = Layout()
        ref.linear_layout_init(ctypes.byref(lo), ctypes.c_longlong(n), ctypes.c_longlong(kb * 2), ctypes.c_longlong(128))
        out = np.empty((n, kb * 2), np.float32)
        st = ref.linear_dequantize_int4(ctypes.byref(lo), ctypes.c_void_p(packed.ctypes.data),
                                        ctypes.c_void_p(scales.ctypes.data), ctypes.c_void_p(out.ctypes.data))
        assert st == 0
        return out

    # all the host threads this process may use, also when a launcher set OMP_NUM_THREADS=1 for its children
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    xt = torch.from_numpy(x)

    def step():
        wgu = torch.from_numpy(dequant(lay.gate_up_packed, lay.gate_up_scales))
        gu = (xt @ wgu.T).to(torch.bfloat16).float()
        g, u = gu[:, :i], gu[:, i:]
        act = ((g / (1 + torch.exp(-g))) * u).to(torch.bfloat16).float()
        wd = torch.from_numpy(dequant(lay.down_packed, lay.down_scales))
        return (act @ wd.T).to(torch.bfloat16)

    for _ in range(min(args.warmup, 2)):
        step()
    steps = min(args.steps, 10)
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    us = (time.perf_counter() - t0) / steps * 1e6
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": round(us, 1), "unit": "us/step", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": round(us / 1e3, 3), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "int4xbf16->f32", "data": "synthetic (seeded numpy)",
        "config": {"workload": f"27B-shape INT4 FFN decode H={h} I={i} M={m} TP=1 on host CPU cores"},
        "cpu_baseline": {"value": round(us, 1), "unit": "us/step", "cores": cores, "kind": kind,
                         "sample": f"{steps} whole steps: dequantize (single thread C) + PyTorch FP32 matmuls ({cores} threads), "
                                   f"os.cpu_count()={os.cpu_count()}"},
        "e2e": {"value": round(us, 1), "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1 only. fused: the cross-rank sum inside the FFN kernel (the product). nccl: comparison "
                         "variant - the same kernel per rank without an exchange, then an NCCL all-reduce of the BF16 "
                         "[M,H] output, which is what the reference's leader all-reduce computes")
    ap.add_argument("--layers", type=int, default=0,
                    help="0: one FFN per step (the headline workload).  L > 0: a step is one pass of h <- h + "
                         "FFN_l(RMSNorm_l(h)) through L independent layers (BASELINE configs[4] at L=64)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
