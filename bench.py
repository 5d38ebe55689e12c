"""Benchmark of the INT4 dense-FFN decode path (metric of BASELINE.json: µs/step and HBM GB/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens M] [--layers L]

N = 1   one 27B-shape FFN (H=5120, I=17408, M=1, TP=1; BASELINE.json configs[2]) per step.
N > 1   launched by torchrun, one rank per GPU: the same layer under tensor parallelism TP=N, every
        rank reading only its slice, the down projection's partial sums reduced inside the kernel
        over NVLink (strong scaling: the total work is fixed).
--layers L   a step is one pass of h <- h + FFN_l(GemmaRMSNorm_l(h)) through L independently
        generated layers (BASELINE configs[4] at L=64); adds the exposed-communication time per step
        (the step minus the same rank's slice run without any exchange) when N > 1.

A step is one call through the C ABI.  Single-layer steps rotate through enough distinct weight
copies that the bytes touched between two uses of one copy exceed twice the L2 (so "HBM GB/s" is an
HBM number); a 64-layer stack is 8.8 GB by itself.  `value` is device time per step with inputs
resident in HBM (K steps captured in one CUDA graph, CUDA events on the launching stream, max over
ranks); `e2e` is the step fed from pinned HOST buffers through ffn_forward_mlp_host, the H2D copy of
x and the D2H copy of y inside the timed region.  `roofline` uses the algorithmic bytes per step per
rank (packed weights + BF16 scales = 1.546875*H*I/TP) against the measured copy peak.  `parity`
is one more call of the same entry point on the CPU oracle's seeded data for the workload just
timed, compared with the oracle at the stated bars (relative L2 <= 5e-3, max-abs <= max(2e-2, one
BF16 ulp)); a failed comparison makes the run exit non-zero.  `cpu_baseline` times the CPU oracle
chain on this box's host cores on a bounded sample.

Comparison variants and side measurements (none of them the headline): --kmajor (the persistent decode
kernel over k-major copies of the down projection), --batched-kernel tcgen05|mma.sync (which pair serves
3..64 tokens), --no-overlap (launches without the dependent-launch attribute), --exchange nccl (N > 1:
the same kernel per rank followed by an NCCL all-reduce), --gemv N,K (one INT4 GEMM call of that
shape), --profile-range (the timed step between cudaProfilerStart/Stop, for a launch list under ncu).

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
TRAFFIC_TABLE = os.path.join(ROOT, "profiles", "dram_traffic_per_launch.json")
STACK_GOLDEN = os.path.join(ROOT, "tests", "golden", "stack_cfg4.npz")


def algorithmic_bytes(h, i, tp):
    return 1.546875 * h * i / tp


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def captured_traffic(tp, tokens, layers):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel from the committed
    table of ncu captures (keyed "tp<TP>_m<M>"); None where that case has no capture."""
    if layers or not os.path.exists(TRAFFIC_TABLE):
        return None
    with open(TRAFFIC_TABLE) as f:
        entry = json.load(f).get(f"tp{tp}_m{tokens}")
    return entry["bytes_per_launch"] if entry else None


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
# parity of the timed workload (the CPU oracle is the checker here, never the thing measured)
# ------------------------------------------------------------------------------------------------
def _bf16_ulp(values):
    import numpy as np
    a = np.abs(values.astype(np.float32))
    return np.exp2(np.floor(np.log2(np.maximum(a, np.float32(2.0 ** -126)))) - 7).astype(np.float64)


def _compare(got, want, rel_bar=5e-3):
    import numpy as np
    g, w = got.astype(np.float64), want.astype(np.float64)
    err = np.abs(g - w)
    rel = float(np.sqrt((err ** 2).sum()) / max(np.sqrt((w ** 2).sum()), 1e-30))
    excess = float(max(0.0, (err - np.maximum(2e-2, _bf16_ulp(want))).max()))
    return {"max_abs": float(err.max()), "rel_l2": rel, "ulp_excess": excess, "over_2e-2": int((err > 2e-2).sum()),
            "rel_l2_bar": rel_bar, "ok": bool(rel <= rel_bar and excess <= 0.0)}


def parity_single_layer(dev, comm, tp, rank, h, i, m, use_nccl, kmajor):
    """One more call of the timed entry point, on the oracle's seeded data of the same shape
    (numpy default_rng: seed 2 up to two tokens as BASELINE configs[2], seed 3 beyond as configs[3]),
    this rank's slice cut by the oracle's slicer, compared with the TP=1 CPU oracle."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from oracle import ffn_oracle as o
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import DenseMlp
    seed = 2 if m <= 2 else 3
    xs, ol = o.draw_config(h, i, seed, tokens=m)
    want = o.ffn(ol[0], xs)
    gp, gs, dp, ds = o.slice_rank(ol[0].gate_up_packed, ol[0].gate_up_scales, ol[0].down_packed, ol[0].down_scales, tp, rank)

    def bits(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.bfloat16)

    mlp = DenseMlp(torch.from_numpy(gp).to(dev), bits(gs), torch.from_numpy(dp).to(dev), bits(ds))
    if kmajor:
        mlp.prepare()
    xd = bits(o.bf16_bits(xs))
    torch.cuda.synchronize()
    if tp > 1:
        dist.barrier()          # the oracle work above takes different host time per rank; the kernel's peer wait is bounded
    if comm is not None:
        out = comm.forward_mlp(mlp, xd)
    else:
        out = mlp.forward_mlp_prepared(xd)
        if use_nccl:
            dist.all_reduce(out)
    L.device_status()
    rep = _compare(out.float().cpu().numpy(), want)
    rep["data"] = f"oracle draw_config({h}, {i}, seed {seed}, tokens {m}), rank slices by the oracle's slicer"
    if tp > 1:
        gathered = [torch.empty_like(out) for _ in range(tp)]
        dist.all_gather(gathered, out)
        rep["ranks_bit_identical"] = all(torch.equal(g.view(torch.int16), out.view(torch.int16)) for g in gathered)
        rep["ok"] = rep["ok"] and rep["ranks_bit_identical"]
    return rep


def parity_stack(dev, layers, comm, tp, h, i, m, x0):
    """The free-running final state of the stack just timed against the committed CPU-oracle
    trajectory (same counter-based weights), within the larger of the per-FFN bar and twice the spread
    between FP32- and FP64-accumulating CPU oracles on this data."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import decode_stack
    if not os.path.exists(STACK_GOLDEN):
        return {"ok": None, "skipped": "no golden trajectory file"}
    g = np.load(STACK_GOLDEN)
    nl, gh, gi, gt, _ = [int(v) for v in g["shape"]]
    if (nl, gh, gi) != (len(layers), h, i) or m > gt:
        return {"ok": None, "skipped": f"the golden trajectory is for {nl} layers of {gh}x{gi}, up to {gt} tokens"}
    want = (g["final_f64"][:m].astype(np.uint32) << 16).view(np.float32)
    spread = float(g["spread_rel_l2"])
    hs = x0.clone()
    torch.cuda.synchronize()
    if tp > 1:
        dist.barrier()
    decode_stack(layers, hs, comm=comm)
    L.device_status()
    rep = _compare(hs.float().cpu().numpy(), want, rel_bar=max(5e-3, 2 * spread))
    rep["ok"] = bool(rep["rel_l2"] <= rep["rel_l2_bar"])      # the chaotic free-running state is gated on relative L2 only
    rep["oracle_vs_oracle_rel_l2"] = spread
    rep["data"] = "free-running final state vs the committed FP64 CPU-oracle trajectory (counter-based weights, seed 4)"
    return rep


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200 import synth
    from haskell_infer_demo_b200.ops import TpComm, bind_forward_mlp_host, decode_stack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L.load()
    if args.no_overlap:
        L.load().ffn_int4_set_launch_overlap(0)
    if args.batched_kernel:
        L.load().ffn_int4_set_batched_kernel({"tcgen05": 0, "mma.sync": 1}[args.batched_kernel])
    tp, m, h, i = world, args.tokens, HIDDEN, INTER
    per_rank_bytes = algorithmic_bytes(h, i, tp)
    stack = args.layers > 0
    # Weights: counter-based synthetic values (N(0, 0.02)-like, see haskell_infer_demo_b200/synth.py), every
    # rank generating and quantizing exactly its own slice on its own device.  Single-layer steps rotate
    # through `copies` DIFFERENT layers; a stack is `--layers` independently generated layers.
    if stack:
        copies = args.layers
        layers = [synth.stack_layer_torch(4, l, h, i, tp, rank, dev) for l in range(copies)]
        x = synth.stack_input_torch(4, m, h, dev)
    else:
        copies = max(2, int(2.2 * L2_BYTES / per_rank_bytes) + 1)
        layers = [synth.stack_layer_torch(2, c, h, i, tp, rank, dev, with_norm=False) for c in range(copies)]
        x = synth.stack_input_torch(2, m, h, dev)
    if args.kmajor:  # k-major copies of the down projections: the decode kernel without the phase barrier
        for lay in layers:
            lay.prepare()
    use_nccl = world > 1 and args.exchange == "nccl"
    if use_nccl and stack:
        raise SystemExit("--exchange nccl is a single-layer comparison; drop --layers")
    comm = TpComm.over_process_group(h, max(m, 2)) if world > 1 and not use_nccl else None
    nl = max(args.layers, 1)
    ws = layers[0].workspace(m)
    out = torch.empty((m, h), dtype=torch.bfloat16, device=dev)
    hstate = x.clone()

    def make_step(with_comm):
        c = comm if with_comm else None

        def step(k):
            if stack:
                hstate.copy_(x)  # restart the residual stream so its magnitude does not drift over the run
                decode_stack(layers, hstate, comm=c, ws=ws, layer_out=out)
                return
            lay = layers[k % copies]
            if c is None:
                lay.forward_mlp_prepared(x, ws=ws, layer_out=out)
                if use_nccl and with_comm:
                    dist.all_reduce(out)
            else:
                c.forward_mlp(lay, x, ws=ws, layer_out=out)
        return step

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def time_steps(step, profiled=False):
        """Warm-up, then K steps captured in one graph; median device time of the replays (ms per K steps)."""
        if profiled:    # `ncu --profile-from-start off` then lists exactly the launches of this function
            torch.cuda.cudart().cudaProfilerStart()
        for k in range(max(args.warmup, 3)):
            step(k)
        barrier()
        L.device_status()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for k in range(args.steps):
                    step(k)
            graph.replay()  # untimed: the first replay uploads the graph
        barrier()
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
        if args.profile_range:
            reps = 2
        for _ in range(reps):
            barrier()
            with torch.cuda.stream(stream):
                e0.record(stream)
                graph.replay()
                e1.record(stream)
            barrier()
            times.append(e0.elapsed_time(e1))
        L.device_status()
        if profiled:
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStop()
        return statistics.median(times), reps, graph

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_total, reps, graph_main = time_steps(make_step(True), profiled=args.profile_range)
    # The same rank's slice with no exchange at all (a TP=1 call on the sliced operands): what the step
    # would cost if communication were free.  exposed communication = step - this.
    ms_alone = None
    if world > 1 and not use_nccl:
        ms_alone, _, graph_alone = time_steps(make_step(False))

    # ---- end to end: host buffers in, host buffer out, every step
    x_host = x.cpu().pin_memory()
    y_host = torch.empty((m, h), dtype=torch.bfloat16).pin_memory()
    staging = torch.empty((2 * m, h), dtype=torch.bfloat16, device=dev)
    x_dev = torch.empty_like(x)
    e2e_steps = args.steps
    cur = torch.cuda.current_stream()
    # the library call with its ctypes arguments built once per layer copy, as a decode loop would hold them
    host_calls = [] if (stack or use_nccl) else [bind_forward_mlp_host(lay, x_host, y_host, staging, ws, comm=comm) for lay in layers]

    def e2e_step(k):
        if stack:
            x_dev.copy_(x_host, non_blocking=True)
            decode_stack(layers, x_dev, comm=comm, ws=ws, layer_out=out)
            y_host.copy_(x_dev, non_blocking=True)
            cur.synchronize()  # the caller needs this step's result before it can issue the next one
        elif use_nccl:
            x_dev.copy_(x_host, non_blocking=True)
            layers[k % copies].forward_mlp_prepared(x_dev, ws=ws, layer_out=out)
            dist.all_reduce(out)
            y_host.copy_(out, non_blocking=True)
            cur.synchronize()
        else:  # ONE library call: copy in, FFN, copy out, one synchronisation
            host_calls[k % copies]()

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
    L.device_status()

    # ---- parity of what was just timed
    parity = None
    if not args.no_parity:
        parity = parity_stack(dev, layers, comm, tp, h, i, m, x) if stack else \
            parity_single_layer(dev, comm, tp, rank, h, i, m, use_nccl, args.kmajor)
        if world > 1 and parity.get("ok") is not None:
            flag = torch.tensor([1 if parity["ok"] else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            parity["ok"] = bool(flag.item())
        if use_nccl:
            parity["note"] = "comparison variant: BF16 partials all-reduced by NCCL; reported, not gated"

    t = torch.tensor([ms_total, e2e_ms, ms_alone or 0.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, ms_alone_max = t.tolist()
    us_step = ms_total * 1e3 / args.steps
    e2e_us = e2e_ms * 1e3 / e2e_steps
    failed = bool(parity and parity.get("ok") is False and not use_nccl)
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        gbs = nl * per_rank_bytes / us_step / 1e3
        kmajor = m <= 2 and args.kmajor   # layers with k-major copies: the persistent decode kernel
        per_layer = 1 if (m <= 2 or kmajor) else (4 if stack else 3)
        launches = nl * per_layer
        if stack and kmajor:
            launches = -(-nl // 64)          # the whole stack in one persistent launch per 64 layers
        line = {
            "metric": METRIC, "value": round(us_step, 3), "unit": "us/step", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(us_step / 1e3, 6),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "int4xbf16->f32",
            "data": "synthetic (counter-based N(0,0.02)-like weights quantized on the device, N(0,1)-like BF16 activations)",
            "tokens_per_s": round(m * 1e6 / us_step, 1),
            "hbm_gbs_per_gpu": round(gbs, 1), "pct_of_8tbs": round(gbs / 80.0, 2),
            "config": {"workload": (f"27B-shape INT4 FFN decode H={h} I={i} M={m} TP={tp} (BASELINE configs[{2 if m <= 2 else 3}])" if not stack else
                                    f"{args.layers}-layer stack h+=FFN(GemmaRMSNorm(h)), {args.layers} independently generated layers, "
                                    f"H={h} I={i} M={m} TP={tp} (BASELINE configs[4])"),
                       "l2": (f"rotating {copies} different layers per rank ({copies * per_rank_bytes / 1e6:.0f} MB > 2x L2)" if not stack else
                              f"{copies} layers = {copies * per_rank_bytes / 1e6:.0f} MB per rank, each read once per step"),
                       "timing": f"{args.steps} steps in one CUDA graph, median of {reps} replays, max over ranks",
                       "launch_overlap": not args.no_overlap},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(gbs / peak, 4), "peak_source": peak_kind, "traffic": captured_traffic(tp, m, args.layers),
                         "algorithmic_bytes_per_launch": per_rank_bytes * nl / launches, "launches_per_step": launches},
            "e2e": {"value": round(e2e_us, 3), "unit": "us/step", "h2d_bytes_per_step": m * h * 2,
                    "d2h_bytes_per_step": m * h * 2,
                    "through": "ffn_forward_mlp_host" if not (stack or use_nccl) else "copy, call, copy, synchronise issued by the caller"},
            "gpu_launches": args.steps * launches,
            "kernel": ("persistent decode kernel over k-major down projections (dp4a)" if kmajor else
                       "row-major single-launch kernel (dp4a)" if m <= 2 else
                       "batched pair (tcgen05, accumulators and converted operand in tensor memory)"
                       if L.load().ffn_int4_set_batched_kernel(-1) == 0 or (L.load().ffn_int4_set_batched_kernel(-1) == 2 and m > 16 and 2 * ((i // tp) // 64) >= 148)
                       else "batched pair (mma.sync bf16)"),
            "exchange": ("none (one GPU)" if world == 1 else "in-kernel tagged-word exchange over NVLink peer memory"
                         if not use_nccl else "comparison variant: NCCL all-reduce of the BF16 output after the kernel"),
            "parity": parity,
            "clocks": clocks,
        }
        if ms_alone is not None:
            alone_us = ms_alone_max * 1e3 / args.steps
            line["exposed_comm"] = {"us_per_step": round(us_step - alone_us, 3), "step_without_exchange_us": round(alone_us, 3),
                                    "how": "the step minus the same rank slice run as a TP=1 call (no exchange), max over ranks"}
        if world == 1 and not args.no_cpu and not stack:
            line["cpu_baseline"] = cpu_baseline(h, i, m, budget_s=12.0)
        print(json.dumps(line), flush=True)
    if comm is not None:
        barrier()
        comm.close()
        dist.destroy_process_group()
    # The comparison variant leaves its process group to interpreter exit: tearing NCCL down while the
    # captured graph that holds its collectives is alive did not return on 8 GPUs.
    if failed:
        sys.exit(3)


# ------------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------------
def host_threads():
    """All the host threads this process may use, also when a launcher set OMP_NUM_THREADS=1 for its children."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return max(1, os.cpu_count() or 1)


def cpu_baseline(h, i, m, budget_s):
    """The oracle chain (FP64-accumulating C loops over the packed bytes; ONE thread by construction)
    on a bounded sample: whole steps of the same workload until the budget is spent."""
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
            "sample": f"{n} whole steps of the same layer (oracle chain from packed bytes, FP64 accumulation, single-threaded C)"}


def run_reference(args):
    """The reference's CPU arithmetic for the path on all host threads: weights dequantized by the
    reference's own linear_dequantize_int4 (oracle/_ref, row blocks spread over the threads; the
    oracle's restatement where that library is absent), FP32 matmuls in PyTorch with the reference's
    three BF16 rounding points.  `value` times a whole step FROM PACKED BYTES (dequantize inside the
    timed region, which is what a CPU has to do with this format); `pre_dequantized` is the same step
    with the FP32 weights prepared beforehand.  Honours --steps / --warmup."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ctypes
    from concurrent.futures import ThreadPoolExecutor

    import numpy as np
    import torch
    from oracle import ffn_oracle as o
    h, i, m = HIDDEN, INTER, args.tokens
    x, layers = o.draw_config(h, i, 2, tokens=m)
    lay = layers[0]
    ref = o.ref_lib()
    kind = "reference" if ref is not None else "port"
    cores = host_threads()
    torch.set_num_threads(cores)
    pool = ThreadPoolExecutor(cores)

    class Layout(ctypes.Structure):
        _fields_ = [(n, ctypes.c_longlong) for n in ("n", "k", "group", "packed_bytes", "scale_count")]

    def dequant_rows(packed, scales, out, r0, r1):
        if ref is None:
            out[r0:r1] = o.dequantize(packed[r0:r1], scales[r0:r1])
            return
        lo = Layout()
        ref.linear_layout_init(ctypes.byref(lo), ctypes.c_longlong(r1 - r0), ctypes.c_longlong(packed.shape[1] * 2), ctypes.c_longlong(128))
        st = ref.linear_dequantize_int4(ctypes.byref(lo), ctypes.c_void_p(packed[r0:r1].ctypes.data),
                                        ctypes.c_void_p(scales[r0:r1].ctypes.data), ctypes.c_void_p(out[r0:r1].ctypes.data))
        assert st == 0

    def dequant(packed, scales):
        n = packed.shape[0]
        out = np.empty((n, packed.shape[1] * 2), np.float32)
        block = max(8, (n // (cores * 4)) // 8 * 8)          # row blocks of whole 8-row tiles; ctypes calls release the GIL
        list(pool.map(lambda r0: dequant_rows(packed, scales, out, r0, min(n, r0 + block)), range(0, n, block)))
        return out

    xt = torch.from_numpy(x)

    def chain(wgu, wd):
        gu = (xt @ wgu.T).to(torch.bfloat16).float()
        g, u = gu[:, :i], gu[:, i:]
        act = ((g / (1 + torch.exp(-g))) * u).to(torch.bfloat16).float()
        return (act @ wd.T).to(torch.bfloat16)

    def step():
        return chain(torch.from_numpy(dequant(lay.gate_up_packed, lay.gate_up_scales)),
                     torch.from_numpy(dequant(lay.down_packed, lay.down_scales)))

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(steps):
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e6)
        return ts

    ts = timed(step, args.steps, args.warmup)
    us = sum(ts) / len(ts)
    wgu = torch.from_numpy(dequant(lay.gate_up_packed, lay.gate_up_scales))
    wd = torch.from_numpy(dequant(lay.down_packed, lay.down_scales))
    tp = timed(lambda: chain(wgu, wd), args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(us, 1), "unit": "us/step", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(us / 1e3, 3), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "int4xbf16->f32", "data": "synthetic (seeded numpy)",
        "config": {"workload": f"27B-shape INT4 FFN decode H={h} I={i} M={m} TP=1 (BASELINE configs[2])",
                   "where": "host CPU cores", "threads": cores, "os_cpu_count": os.cpu_count()},
        "cpu_baseline": {"value": round(us, 1), "unit": "us/step", "cores": cores, "kind": kind,
                         "sample": f"{args.steps} whole steps from packed bytes: dequantize ({'reference C' if ref is not None else 'oracle C'}, "
                                   f"row blocks over {cores} threads) + PyTorch FP32 matmuls ({cores} threads)",
                         "median_us": round(statistics.median(ts), 1), "min_us": round(min(ts), 1), "max_us": round(max(ts), 1)},
        "pre_dequantized": {"value": round(sum(tp) / len(tp), 1), "unit": "us/step", "median_us": round(statistics.median(tp), 1),
                            "min_us": round(min(tp), 1), "max_us": round(max(tp), 1),
                            "what": "the same step with the FP32 weights dequantized beforehand (1.07 GB resident)"},
        "e2e": {"value": round(us, 1), "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# the other decode GEMVs of the format (single-matrix mode of the streaming kernel)
# ------------------------------------------------------------------------------------------------
def run_gemv(args):
    """`--gemv N,K`: device time of one INT4 GEMV/GEMM call (ffn_gemm_int4_bf16, M = --tokens) on an [N, K]
    matrix - attention projections, the LM head - rotating through weight copies larger than 2x L2.
    One JSON line; a side measurement, not the headline metric."""
    import ctypes
    import torch
    from haskell_infer_demo_b200 import lib as L
    n, k = (int(v) for v in args.gemv.split(","))
    m = args.tokens
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    lib = L.load()
    bytes_per = n * k // 2 + n * (k // 128) * 2
    copies = max(2, int(2.2 * L2_BYTES / bytes_per) + 1)
    ws = [(torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev) & 0x77,
           torch.full((n, k // 128), 0.01, dtype=torch.bfloat16, device=dev)) for _ in range(copies)]
    x = torch.randn((m, k), device=dev).to(torch.bfloat16)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.Stream()

    def call(c):
        p, sc = ws[c % copies]
        L.check(lib.ffn_gemm_int4_bf16(x.data_ptr(), p.data_ptr(), sc.data_ptr(), out.data_ptr(), m, n, k, 128,
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    with torch.cuda.stream(stream):
        for c in range(max(args.warmup, 3)):
            call(c)
    torch.cuda.synchronize()
    L.device_status()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for c in range(args.steps):
                call(c)
        graph.replay()
    torch.cuda.synchronize()
    e0, e1, ts = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), []
    for _ in range(20):
        with torch.cuda.stream(stream):
            e0.record(stream)
            graph.replay()
            e1.record(stream)
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / args.steps)
    L.device_status()
    us = statistics.median(ts)
    peak, peak_kind = measured_peak_gbs()
    plan = ctypes.create_string_buffer(1024)
    lib.ffn_int4_describe_gemm_plan(m, n, k, 148, 232448, plan, 1024)
    print(json.dumps({"metric": "int4_gemm_latency", "value": round(us, 3), "unit": "us/call", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "higher_is_better": False, "dtype": "int4 weights x bf16 activations, fp32 accumulate",
                      "data": "synthetic", "config": {"workload": f"INT4 GEMM M={m} N={n} K={k}", "l2": f"rotating {copies} copies",
                                                     "plan": plan.value.decode()},
                      "roofline": {"bound": "hbm", "achieved": round(bytes_per / us / 1e3, 1), "peak": peak, "unit": "GB/s",
                                   "frac": round(bytes_per / us / 1e3 / peak, 4), "peak_source": peak_kind},
                      "gpu_launches": args.steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison of the timed workload")
    ap.add_argument("--kmajor", action="store_true",
                    help="comparison variant: register k-major copies of the down projections, so that one or two tokens "
                         "run the persistent decode kernel (a whole stack in one launch) instead of the row-major "
                         "single-launch kernel, which measured faster and is the default")
    ap.add_argument("--batched-kernel", default="", choices=["", "tcgen05", "mma.sync"],
                    help="3..64 tokens: which pair of kernels runs (default: the library's own choice)")
    ap.add_argument("--profile-range", action="store_true",
                    help="for a launch list under `ncu --profile-from-start off`: the warm-up and the timed graph replays "
                         "(two of them instead of about 0.6 s worth) run between cudaProfilerStart and cudaProfilerStop; "
                         "numbers printed by such a run are not bench values")
    ap.add_argument("--no-overlap", action="store_true",
                    help="comparison variant: launch without the programmatic-dependent-launch attribute")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1 only. fused: the cross-rank sum inside the FFN kernel (the product). nccl: comparison "
                         "variant - the same kernel per rank without an exchange, then an NCCL all-reduce of the BF16 "
                         "[M,H] output, which is what the reference's leader all-reduce computes")
    ap.add_argument("--layers", type=int, default=0,
                    help="0: one FFN per step (the headline workload).  L > 0: a step is one pass of h <- h + "
                         "FFN_l(RMSNorm_l(h)) through L independent layers (BASELINE configs[4] at L=64)")
    ap.add_argument("--gemv", default="", help="N,K: time one INT4 GEMM call of that shape instead of the FFN (side measurement)")
    args = ap.parse_args()
    if args.gemv:
        run_gemv(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
