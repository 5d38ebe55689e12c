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
           os.path.join(ROOT, "tests", "tp_worker.py"), "0:1", "0:2", "0:8", "0:16", "1:1", "1:64"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert proc.returncode == 0 and "tp_worker ok" in proc.stdout, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.parametrize("tokens", [1, 8])
def test_withheld_rank_is_reported_not_waited_for_forever(cuda, tokens):
    """Failure detection without a GPU fault: rank 0 of a two-rank communicator runs alone (rank 1 is
    never launched, so its partial sums never arrive).  The kernel's wait for them is bounded (about
    a second); it must return, the host must see the status naming the wait, and the device must
    stay usable: the next plain call gives the right answer.  Covers the single-pass kernel and the
    batched pair."""
    from oracle import ffn_oracle as o
    from gpu_util import assert_ffn_close, dev_bf16, host_f32, upload_layer
    from haskell_infer_demo_b200 import lib as L
    from haskell_infer_demo_b200.ops import TpComm
    x, layers = o.draw_config(1024, 3072, 0, tokens=tokens)
    comms = TpComm.local([cuda, cuda], 1024, 8)      # both ends on this device; only rank 0 is driven
    try:
        half = upload_layer(layers[0], cuda, tp=2, rank=0)
        comms[0].forward_mlp(half, dev_bf16(x, cuda))
        with pytest.raises(L.FfnError, match="partial sums"):
            L.device_status()
        L.device_status()                            # the status was cleared by reading it
        whole = upload_layer(layers[0], cuda)
        got = host_f32(whole.forward_mlp_prepared(dev_bf16(x, cuda)))
        L.device_status()
        assert_ffn_close(got, o.ffn(layers[0], x), "after a withheld rank")
    finally:
        for c in comms:
            c.close()
