"""Host-side mirror of the reference's operator interface for the INT4 FFN path, over torch CUDA
tensors.  Each function validates nothing itself: arguments go to the C ABI unchanged and the
library's status/last-error is raised as :class:`FfnError`, so error behaviour is the library's.

Names follow the reference: ``gemm_int4_bf16`` (csrc/include/layers.h:376), ``forward_mlp`` /
``forward_mlp_prepared`` (layers.h:330-337), ``kernel_silu_mul_packed`` (kernels.h),
``kernel_gemma_rms_norm``, ``kernel_residual_add``.
"""
import ctypes

import torch

from .lib import MlpWeights, ModelDims, check, load

GROUP = 128


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("this path runs on CUDA tensors only; there is no CPU implementation")


def gemm_int4_bf16(a, packed, scales, group=GROUP):
    """a bf16 [M, K]; packed uint8 [N, K/2]; scales bf16-bits (int16/uint16/bfloat16) [N, K/128]
    -> bf16 [M, N]."""
    _require_cuda(a, packed, scales)
    m, k = a.shape
    n = packed.shape[0]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    check(load().ffn_gemm_int4_bf16(_ptr(a), _ptr(packed), _ptr(scales), _ptr(out), m, n, k, group,
                                    _stream()))
    return out


def kernel_silu_mul_packed(packed_act):
    """bf16 [T, 2I] (gate half then up half per row) -> bf16 [T, I]."""
    _require_cuda(packed_act)
    t, two_i = packed_act.shape
    out = torch.empty((t, two_i // 2), dtype=torch.bfloat16, device=packed_act.device)
    check(load().ffn_silu_mul_packed(_ptr(out), _ptr(packed_act), t, two_i // 2, _stream()))
    return out


def kernel_gemma_rms_norm(x, weight, eps=1e-6):
    _require_cuda(x, weight)
    rows, cols = x.shape
    out = torch.empty_like(x)
    check(load().ffn_gemma_rms_norm(_ptr(out), _ptr(x), _ptr(weight), cols, rows, eps, _stream()))
    return out


def kernel_residual_add(dst, src):
    _require_cuda(dst, src)
    check(load().ffn_residual_add(_ptr(dst), _ptr(src), dst.numel(), _stream()))
    return dst


def quantize_int4(weights):
    """FP32 [N, K] on the device -> (packed u8 [N, K/2], scales bf16 [N, K/128]), the bytes the
    reference's quantizer writes (include/ffn_int4.h, ffn_quantize_int4)."""
    _require_cuda(weights)
    if weights.dtype != torch.float32 or weights.dim() != 2 or not weights.is_contiguous():
        raise ValueError("quantize_int4 takes a contiguous FP32 [N, K] tensor")
    n, k = weights.shape
    packed = torch.empty((n, k // 2), dtype=torch.uint8, device=weights.device)
    scales = torch.empty((n, k // 128), dtype=torch.bfloat16, device=weights.device)
    check(load().ffn_quantize_int4(_ptr(weights), _ptr(packed), _ptr(scales), n, k, _stream()))
    return packed, scales


def dequantize_int4(packed, scales):
    """float(code) * float(scale) through the kernels' unpack routine -> (fp32 [N, K], count of
    reserved 0x8 nibbles)."""
    _require_cuda(packed, scales)
    n, kb = packed.shape
    out = torch.empty((n, kb * 2), dtype=torch.float32, device=packed.device)
    bad = torch.zeros(1, dtype=torch.int32, device=packed.device)
    check(load().ffn_dequantize_int4(_ptr(out), _ptr(packed), _ptr(scales), n, kb * 2, _ptr(bad),
                                     _stream()))
    return out, int(bad.item())


class DenseMlp:
    """One layer's (rank-local) INT4 operands on the device, shaped like the reference's
    MlpWeights: gate_up [2I, H/2] u8 + scales [2I, H/128], down [H, I/2] u8 + scales [H, I/128],
    optional post-norm weight bf16 [H]."""

    def __init__(self, gate_up, gate_up_scales, down, down_scales, post_norm_w=None, rms_eps=1e-6,
                 max_chunk=128):
        _require_cuda(gate_up, gate_up_scales, down, down_scales, post_norm_w)
        self.tensors = (gate_up, gate_up_scales, down, down_scales, post_norm_w)  # keep alive
        self.hidden = gate_up.shape[1] * 2
        self.inter = gate_up.shape[0] // 2
        self.weights = MlpWeights(0, 0, 0, post_norm_w.data_ptr() if post_norm_w is not None else 0,
                                  gate_up.data_ptr(), gate_up_scales.data_ptr(), down.data_ptr(),
                                  down_scales.data_ptr(), GROUP)
        self.dims = ModelDims()
        self.dims.hidden_size = self.hidden
        self.dims.intermediate_size = self.inter
        self.dims.norm_style = 0
        self.dims.rms_eps = rms_eps
        self.dims.max_chunk = max_chunk
        self.device = gate_up.device

    def prepare(self):
        """Register the k-major copy of this layer's down projection (include/ffn_int4.h,
        ffn_decode_layer_prepare): decode calls of 1-2 tokens then take the kernel without the phase
        barrier, and decode_stack runs in one persistent launch.  Released when the object dies."""
        check(load().ffn_decode_layer_prepare(ctypes.byref(self.weights), ctypes.byref(self.dims), _stream()))
        self.prepared = True
        return self

    def release(self):
        if getattr(self, "prepared", False):
            load().ffn_decode_layer_release(ctypes.byref(self.weights))
            self.prepared = False

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    def workspace(self, tokens):
        """The reference's layer workspace for the MLP: tokens*(H+3I) bf16 (layers.cu:65)."""
        return torch.empty(tokens * (self.hidden + 3 * self.inter), dtype=torch.bfloat16,
                           device=self.device)

    def forward_mlp(self, residual, ws=None, layer_out=None):
        """norm (when the layer has a post-norm weight) + FFN; returns layer_out bf16 [T, H]."""
        tokens = residual.shape[0]
        ws = self.workspace(tokens) if ws is None else ws
        layer_out = torch.empty((tokens, self.hidden), dtype=torch.bfloat16,
                                device=self.device) if layer_out is None else layer_out
        check(load().ffn_forward_mlp(None, _stream(), _ptr(residual), _ptr(ws), _ptr(layer_out),
                                     ctypes.byref(self.weights), tokens, ctypes.byref(self.dims)))
        return layer_out

    def forward_mlp_prepared(self, normed, ws=None, layer_out=None):
        tokens = normed.shape[0]
        ws = self.workspace(tokens) if ws is None else ws
        layer_out = torch.empty((tokens, self.hidden), dtype=torch.bfloat16,
                                device=self.device) if layer_out is None else layer_out
        check(load().ffn_forward_mlp_prepared(None, _stream(), _ptr(normed), _ptr(ws), _ptr(layer_out),
                                              ctypes.byref(self.weights), tokens,
                                              ctypes.byref(self.dims)))
        return layer_out


class TpComm:
    """One rank's end of the in-kernel cross-rank reduce (include/ffn_int4.h, ffn_tp_*).

    ``TpComm.over_process_group(hidden, max_tokens)`` is the one-process-per-GPU form: each rank
    allocates its exchange buffer, the CUDA IPC handles travel through torch.distributed, and every
    rank maps every peer's buffer.  ``TpComm.local(devices, ...)`` is the reference's process model
    (one process drives every rank) and returns one communicator per device.
    """

    def __init__(self, handle, tp, rank):
        self.handle, self.tp, self.rank = handle, tp, rank

    @staticmethod
    def _create(tp, rank, hidden, max_tokens):
        h = ctypes.c_void_p()
        check(load().ffn_tp_create(ctypes.byref(h), tp, rank, hidden, max_tokens))
        return TpComm(h, tp, rank)

    @classmethod
    def over_process_group(cls, hidden, max_tokens, group=None):
        import torch.distributed as dist
        tp, rank = dist.get_world_size(group), dist.get_rank(group)
        comm = cls._create(tp, rank, hidden, max_tokens)
        if tp > 1:
            mine = (ctypes.c_uint8 * 64)()
            check(load().ffn_tp_export(comm.handle, mine))
            gathered = [None] * tp
            dist.all_gather_object(gathered, bytes(mine), group=group)
            blob = b"".join(gathered)
            check(load().ffn_tp_connect(comm.handle, ctypes.c_char_p(blob)))
            dist.barrier(group)
        return comm

    @classmethod
    def local(cls, devices, hidden, max_tokens):
        comms = []
        for r, d in enumerate(devices):
            with torch.cuda.device(d):
                comms.append(cls._create(len(devices), r, hidden, max_tokens))
        if len(devices) > 1:
            arr = (ctypes.c_void_p * len(devices))(*[c.handle for c in comms])
            check(load().ffn_tp_connect_local(arr, len(devices)))
        return comms

    def forward_mlp(self, mlp, normed, ws=None, layer_out=None, residual=None):
        """``mlp`` holds this rank's slice (see DenseMlp); returns the reduced bf16 [T, H]."""
        tokens = normed.shape[0]
        ws = mlp.workspace(tokens) if ws is None else ws
        layer_out = torch.empty((tokens, mlp.hidden), dtype=torch.bfloat16,
                                device=mlp.device) if layer_out is None else layer_out
        check(load().ffn_forward_mlp_tp(self.handle, _stream(), _ptr(normed), _ptr(ws), _ptr(layer_out),
                                        ctypes.byref(mlp.weights), tokens, ctypes.byref(mlp.dims),
                                        _ptr(residual)))
        return layer_out

    def close(self):
        if self.handle:
            load().ffn_tp_destroy(self.handle)
            self.handle = None


def decode_stack(mlps, h, comm=None, ws=None, layer_out=None):
    """h <- h + FFN_l(RMSNorm_l(h)) over the layers in ``mlps`` (DenseMlp objects with a post-norm
    weight), in place; ``comm`` is a TpComm (None = TP 1).  Returns h."""
    tokens = h.shape[0]
    first = mlps[0]
    ws = first.workspace(tokens) if ws is None else ws
    layer_out = torch.empty((tokens, first.hidden), dtype=torch.bfloat16,
                            device=first.device) if layer_out is None else layer_out
    arr = (MlpWeights * len(mlps))(*[m.weights for m in mlps])
    check(load().ffn_decode_stack(comm.handle if comm is not None else None, _stream(), _ptr(h), _ptr(ws),
                                  _ptr(layer_out), arr, len(mlps), tokens, ctypes.byref(first.dims)))
    return h


def forward_mlp_host(mlp, normed_host, layer_out_host, staging, ws, comm=None):
    """One FFN for activations in (pinned) HOST memory: copy in, FFN, copy out and one stream
    synchronisation inside a single library call (include/ffn_int4.h, ffn_forward_mlp_host).
    ``staging`` is device memory for 2*T*H bf16; ``comm`` a TpComm (None = TP 1)."""
    tokens = normed_host.shape[0]
    check(load().ffn_forward_mlp_host(comm.handle if comm is not None else None, _stream(),
                                      ctypes.c_void_p(normed_host.data_ptr()), ctypes.c_void_p(layer_out_host.data_ptr()),
                                      _ptr(staging), _ptr(ws), ctypes.byref(mlp.weights), tokens, ctypes.byref(mlp.dims)))
    return layer_out_host


def bind_forward_mlp_host(mlp, normed_host, layer_out_host, staging, ws, comm=None):
    """forward_mlp_host with its arguments converted once: returns a zero-argument callable that makes
    exactly the C call (a decode loop calls the same buffers every step; building eight ctypes
    objects per call costs about 5 us of the 52 the call takes)."""
    fn = load().ffn_forward_mlp_host
    args = (comm.handle if comm is not None else None, _stream(), ctypes.c_void_p(normed_host.data_ptr()),
            ctypes.c_void_p(layer_out_host.data_ptr()), _ptr(staging), _ptr(ws), ctypes.byref(mlp.weights),
            normed_host.shape[0], ctypes.byref(mlp.dims))
    keep = (mlp, normed_host, layer_out_host, staging, ws, comm)     # the buffers must outlive the callable

    def call():
        st = fn(*args)
        if st:
            check(st)
        return keep[2]
    return call


def tp_allreduce_sum(comm, buffer):
    """In-place sum of ``buffer`` (bf16 or fp32, at most max_tokens*hidden elements) over the ranks of
    ``comm`` through the exchange slots (include/ffn_int4.h, ffn_tp_allreduce_sum)."""
    _require_cuda(buffer)
    dtype = {torch.float32: 0, torch.bfloat16: 2}[buffer.dtype]
    check(load().ffn_tp_allreduce_sum(comm.handle, _stream(), _ptr(buffer), buffer.numel(), dtype))
    return buffer
