"""Worker for the tensor-parallel GPU parity test: run under torch.distributed.run, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node R --master-addr 127.0.0.1 \
        --master-port 29531 tests/tp_worker.py [cfg ...]

Every rank draws the same seeded configuration, keeps its slice (gate/up rows, down columns, global
scales), runs the FFN with the in-kernel cross-rank reduce and checks: (1) the result against the
TP=1 CPU oracle at the stated bars, (2) bit-identical results on every rank, (3) repeatability over
many back-to-back calls (the exchange slots are reused), (4) the fused residual update.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import ffn_oracle as o  # noqa: E402
from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer  # noqa: E402
from haskell_infer_demo_b200 import lib as L  # noqa: E402
from haskell_infer_demo_b200.ops import TpComm  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    args = [a for a in sys.argv[1:] if ":" in a]
    flags = [a for a in sys.argv[1:] if ":" not in a]
    cases = [(int(a.split(":")[0]), int(a.split(":")[1])) for a in args] or [(0, 1), (0, 2), (1, 1)]
    comms = {}
    drawn = {}
    for cfg, tokens in cases:
        spec = o.CONFIGS[cfg]
        h, i = spec["hidden"], spec["inter"]
        if (i // world) % 128:
            if rank == 0:
                print(f"config {cfg}: I/{world} is not a whole number of groups, skipped")
            continue
        if cfg not in drawn:
            # one draw per configuration, with as many activation rows as its largest case; a case
            # of fewer tokens takes the first rows (drawing 267 M weights costs seconds of host time
            # on every rank while the GPUs wait)
            most = max(t for c, t in cases if c == cfg)
            xs, layers = o.draw_config(h, i, spec["seed"], tokens=most)
            drawn.clear()
            drawn[cfg] = (xs, layers[0], upload_layer(layers[0], dev, tp=world, rank=rank))
        xs, layer0, mlp = drawn[cfg]
        layers = [layer0]
        x = xs[:tokens]
        want = o.ffn(layers[0], x)
        if h not in comms:
            comms[h] = TpComm.over_process_group(h, 64)
        comm = comms[h]
        xd = dev_bf16(x, dev)
        dist.barrier()      # host-side oracle work differs per rank; the kernel's peer wait is bounded (~0.2 s)
        got_t = comm.forward_mlp(mlp, xd)
        L.device_status()
        got = host_f32(got_t)
        max_abs, rel = assert_ffn_close(got, want, f"config {cfg} M={tokens} TP={world} rank {rank}")
        # identical on every rank
        gathered = [torch.empty_like(got_t) for _ in range(world)]
        dist.all_gather(gathered, got_t)
        for r in range(world):
            assert torch.equal(gathered[r].view(torch.int16), got_t.view(torch.int16)), f"rank {r} differs"
        # repeatable: the exchange slots are reused call after call
        for _ in range(25):
            again = comm.forward_mlp(mlp, xd)
        L.device_status()
        assert torch.equal(again.view(torch.int16), got_t.view(torch.int16))
        # fused residual update: h <- bf16(h + y)
        hres = o.bf16_round(np.random.default_rng(5).standard_normal((tokens, h), dtype=np.float32))  # residual stream
        res = dev_bf16(hres, dev)
        y = comm.forward_mlp(mlp, xd, residual=res)
        L.device_status()
        assert torch.equal(y.view(torch.int16), got_t.view(torch.int16))
        assert np.array_equal(host_f32(res), o.residual_add(hres, got))
        if rank == 0:
            note = ""
            if tokens <= 2:     # the emulation of the reference's own TP arithmetic costs host seconds per token
                ref_tp = o.ffn_reference_tp(layers[0], x, world)
                note = f" (the reference's BF16 leader reduce would sit at rel-L2 {o.compare(ref_tp, want)[1]:.3g})"
            print(f"config {cfg} M={tokens} TP={world}: max-abs {max_abs:.3g} rel-L2 {rel:.3g}{note}", flush=True)
    drawn.clear()
    if "stack64" in flags:
        # BASELINE configs[4] at its full shape: 64 independently generated layers, this rank's slices
        # made on its own device, checked against the committed CPU-oracle trajectory
        from haskell_infer_demo_b200 import synth
        from test_stack_gpu import check_stack_against_golden, load_stack_golden
        golden = load_stack_golden()
        nl, hidden, inter, _, seed = [int(v) for v in golden["shape"]]
        if (inter // world) % 128 == 0:
            mlps = [synth.stack_layer_torch(seed, l, hidden, inter, world, rank, dev) for l in range(nl)]
            if hidden not in comms:
                comms[hidden] = TpComm.over_process_group(hidden, 64)
            res = check_stack_against_golden(dev, mlps, golden, comm=comms[hidden], sync=dist.barrier, what=f"TP={world}")
            for m, (rel, h) in res.items():
                gathered = [torch.empty_like(h) for _ in range(world)]
                dist.all_gather(gathered, h)
                for r in range(world):
                    assert torch.equal(gathered[r].view(torch.int16), h.view(torch.int16)), f"rank {r} differs"
            del mlps
    # config-4 style stack under TP: norm + FFN + reduce + residual per layer, all ranks identical
    from haskell_infer_demo_b200.ops import decode_stack
    for tokens in (1, 8, 2):      # single-pass and batched kernels alternate on one communicator
        hidden, inter, nl = 1024, 3072, 6
        if (inter // world) % 128:
            break
        h0, layers = o.draw_config(hidden, inter, 4, tokens=tokens, layers=nl, with_norm=True)
        ref = o.stack(layers, h0)
        mlps = [upload_layer(lay, dev, tp=world, rank=rank, with_norm=True) for lay in layers]
        if hidden not in comms:
            comms[hidden] = TpComm.over_process_group(hidden, 64)
        inputs = [h0] + ref[:-1]
        for l in range(nl):                       # teacher-forced per layer
            h = dev_bf16(inputs[l], dev).clone()
            dist.barrier()
            decode_stack([mlps[l]], h, comm=comms[hidden])
            L.device_status()
            assert_ffn_close(host_f32(h), ref[l], f"stack layer {l} M={tokens} TP={world}")
        h = dev_bf16(h0, dev).clone()
        dist.barrier()
        decode_stack(mlps, h, comm=comms[hidden])
        L.device_status()
        gathered = [torch.empty_like(h) for _ in range(world)]
        dist.all_gather(gathered, h)
        for r in range(world):
            assert torch.equal(gathered[r].view(torch.int16), h.view(torch.int16)), f"rank {r} differs"
        if rank == 0:
            print(f"stack M={tokens} TP={world}: free-running rel-L2 {o.compare(host_f32(h), ref[-1])[1]:.3g}", flush=True)
    dist.barrier()
    for c in comms.values():
        c.close()
    dist.destroy_process_group()
    if rank == 0:
        print("tp_worker ok", flush=True)


if __name__ == "__main__":
    main()
