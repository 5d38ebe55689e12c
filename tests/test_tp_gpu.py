"""Tensor-parallel parity on real GPUs: needs two or more devices, otherwise skips itself (as the
reference's collective test does, tests/kernels/test_collective.cu:125-128).  Ranks run as
torch.distributed.run children over NCCL-free peer memory (NCCL only carries the handle exchange)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_tp1_communicator_matches_plain_call(cuda):
    """TP=1 through the communicator entry point is the plain fused FFN."""
    from oracle import ffn_oracle as o
    from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import TpComm
    x, layers = o.draw_config(1024, 3072, 0)
    mlp = upload_layer(layers[0], cuda)
    comm = TpComm.local([cuda], 1024, 2)[0]
    try:
        got = comm.forward_mlp(mlp, dev_bf16(x, cuda))
        L.device_status()
        plain = mlp.forward_mlp_prepared(dev_bf16(x, cuda))
        assert torch.equal(got.view(torch.int16), plain.view(torch.int16))
        assert_ffn_close(host_f32(got), o.ffn(layers[0], x), "TP=1 communicator")
    finally:
        comm.close()


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_tp_parity_multi_gpu(ranks):
    if not torch.cuda.is_available() or torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
           "--master-addr", "127.0.0.1", "--master-port", str(29530 + ranks),
           os.path.join(ROOT, "tests", "tp_worker.py"), "0:1", "0:2", "0:8", "0:16", "1:1", "1:64",
           # the shapes the benchmark is quoted on (BASELINE configs[2], [3], [4]): H=5120, I=17408
           "2:1", "2:2", "2:16", "3:16", "3:32", "3:64", "stack64"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env, cwd=ROOT)
    assert proc.returncode == 0 and "tp_worker ok" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.parametrize("tokens,kmajor", [(1, False), (8, False), (1, True), (2, True)])
def test_withheld_rank_is_reported_not_waited_for_forever(cuda, tokens, kmajor):
    """Failure detection without a GPU fault: rank 0 of a two-rank communicator runs alone (rank 1 is
    never launched, so its partial sums never arrive).  The kernel's wait for them is bounded (about
    a second); it must return, the host must see the status naming the wait, and the device must
    stay usable: the next plain call gives the right answer.  Covers the row-major single-pass kernel,
    the batched pair and the kernel over k-major copies."""
    from oracle import ffn_oracle as o
    from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import TpComm
    x, layers = o.draw_config(1024, 3072, 0, tokens=tokens)
    comms = TpComm.local([cuda, cuda], 1024, 8)      # both ends on this device; only rank 0 is driven
    try:
        half = upload_layer(layers[0], cuda, tp=2, rank=0, prepare=kmajor)
        comms[0].forward_mlp(half, dev_bf16(x, cuda))
        with pytest.raises(L.FfnError, match="partial sums"):
            L.device_status()
        L.device_status()                            # the status was cleared by reading it
        whole = upload_layer(layers[0], cuda, prepare=kmajor)
        got = host_f32(whole.forward_mlp_prepared(dev_bf16(x, cuda)))
        L.device_status()
        assert_ffn_close(got, o.ffn(layers[0], x), "after a withheld rank")
    finally:
        for c in comms:
            c.close()


def _local_ranks():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 0


def test_one_process_drives_every_rank_like_the_reference(cuda):
    """The reference's process model (csrc/include/engine.h:8-9; forward_replicated,
    csrc/engine.cu:1603-1657): ONE host thread issues every rank's launch in rank order, each on its own
    device and stream, and synchronises afterwards.  Communicators wired with ffn_tp_connect_local (peer
    access, no IPC).  Every rank's kernel waits (bounded) for the others' partial sums, so this only works
    because launches are asynchronous - which is what the test pins, on the small shape and on the 27B
    shape, for the single-launch kernel and the tensor-core pair, with results equal to the oracle and
    bit-identical on all ranks."""
    from oracle import ffn_oracle as o
    from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import TpComm
    ranks = _local_ranks()
    if not ranks:
        pytest.skip("needs two or more GPUs")
    devices = [torch.device("cuda", r) for r in range(ranks)]
    for hidden, inter, seed in ((1024, 3072, 0), (5120, 17408, 2)):
        if (inter // ranks) % 128:
            continue
        xs, layers = o.draw_config(hidden, inter, seed, tokens=16)
        comms = TpComm.local(devices, hidden, 16)
        try:
            mlps = [upload_layer(layers[0], d, tp=ranks, rank=r) for r, d in enumerate(devices)]
            for tokens, kmajor in ((1, False), (2, False), (16, False), (1, True), (2, True)):
                if kmajor:                                            # over the k-major copies of the down slices
                    for r, d in enumerate(devices):
                        with torch.cuda.device(d):
                            mlps[r].prepare()
                x = xs[:tokens]
                want = o.ffn(layers[0], x)
                xd = [dev_bf16(x, d) for d in devices]
                for d in devices:
                    torch.cuda.synchronize(d)
                for rep in range(3):                                  # slots are reused call after call
                    outs = []
                    for r, d in enumerate(devices):                   # one thread, rank order, no sync in between
                        with torch.cuda.device(d):
                            outs.append(comms[r].forward_mlp(mlps[r], xd[r]))
                    for d in devices:
                        with torch.cuda.device(d):
                            L.device_status()
                    assert_ffn_close(host_f32(outs[0]), want, f"one process, {ranks} ranks, H={hidden} M={tokens} k-major={kmajor}")
                    for r in range(1, ranks):
                        assert torch.equal(outs[r].cpu().view(torch.int16), outs[0].cpu().view(torch.int16)), f"rank {r} differs"
        finally:
            for c in comms:
                c.close()


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_allreduce_sum_entry_exact_by_construction(cuda, dtype):
    """ffn_allreduce_sum (the allreduce_sum-shaped entry) on small integers, exact in every element
    type, as the reference's collective test does (tests/kernels/test_collective.cu:68-117), with the
    buffers overwritten between back-to-back rounds (its race test, :214-269)."""
    import ctypes
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import TpComm
    ranks = _local_ranks()
    if not ranks:
        pytest.skip("needs two or more GPUs")
    devices = [torch.device("cuda", r) for r in range(ranks)]
    hidden, rows = 1024, 8
    comms = TpComm.local(devices, hidden, rows)
    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    try:
        n = hidden * rows - 13                                       # a ragged count
        for rnd in range(8):
            bufs = [((torch.arange(n, device=d) % 7) + r + rnd).to(td) for r, d in enumerate(devices)]
            want = sum(((torch.arange(n) % 7) + r + rnd).float() for r in range(ranks))
            for d in devices:
                torch.cuda.synchronize(d)
            arr_c = (ctypes.c_void_p * ranks)(*[c.handle for c in comms])
            arr_s = (ctypes.c_void_p * ranks)(*[torch.cuda.current_stream(d).cuda_stream for d in devices])
            arr_b = (ctypes.c_void_p * ranks)(*[b.data_ptr() for b in bufs])
            L.check(L.load().ffn_allreduce_sum(arr_c, arr_s, ranks, arr_b, n, 2 if dtype == "bf16" else 0))
            for d in devices:
                with torch.cuda.device(d):
                    L.device_status()
            for b in bufs:
                assert torch.equal(b.float().cpu(), want)
        assert L.load().ffn_allreduce_sum(arr_c, arr_s, ranks, arr_b, n, 1) == -4        # f16: not a type this entry takes
        assert L.load().ffn_allreduce_sum(arr_c, arr_s, ranks, arr_b, hidden * rows + 1, 0) == -4
    finally:
        for c in comms:
            c.close()
