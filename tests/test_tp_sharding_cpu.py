"""World-size-2 (gloo, CPU) check of the tensor-parallel sharding the N>1 path relies on: each rank
keeps its slice with the GLOBAL scales, computes its FP32 partial of the down projection, the ranks'
partials are summed in rank order and rounded once - and that equals the TP=1 oracle.  This is the
host-side half of the fused reduce (the device half needs GPUs, tests/test_tp_gpu.py)."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from oracle import ffn_oracle as o
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, layers = o.draw_config(512, 1024, 11, tokens=2)
    lay = layers[0]
    gp, gs, dp, ds = o.slice_rank(lay.gate_up_packed, lay.gate_up_scales, lay.down_packed, lay.down_scales,
                                  world, rank)
    gu = o.bf16_round(o.matmul_packed_f64(x, gp, gs).astype(np.float32))
    half = gu.shape[1] // 2
    act = o.silu_mul(gu[:, :half], gu[:, half:])
    partial = torch.from_numpy(o.matmul_packed_f64(act, dp, ds).astype(np.float32))
    slots = [torch.empty_like(partial) for _ in range(world)]
    dist.all_gather(slots, partial)          # every rank holds every rank's slot, as the kernel's peers do
    total = slots[0].clone()
    for r in range(1, world):                # fixed rank order -> identical bits on every rank
        total += slots[r]
    y = o.bf16_round(total.numpy())
    want = o.ffn(lay, x)
    max_abs, rel = o.compare(y, want)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y)
    assert rel <= 5e-3 and max_abs <= 2e-2, (max_abs, rel)
    dist.destroy_process_group()


def test_rank_order_sum_of_sliced_partials_matches_tp1_oracle(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    y0, y1 = np.load(tmp_path / "y0.npy"), np.load(tmp_path / "y1.npy")
    assert np.array_equal(y0, y1)
