"""Counter-based synthetic weights: the same bits on the CPU (numpy) and on the GPU (torch).

The reference's own tests build synthetic checkpoints (tests/synth/make_qwen3_dense.py) and
deterministic index-hash fixtures (tests/kernels/test_utils.h:57-63) where real checkpoints are too
large to carry.  The 64-layer 27B-shape stack has 17 G weights: drawing them with a sequential
generator takes minutes of host time per run, so they are defined here as a pure function of
(seed, tensor, layer, element index) that any machine can evaluate for any slice:

    z      = splitmix64(key(seed, tensor, layer) + index)
    s      = sum of the four 16-bit fields of z, minus 131070        integer in [-131070, 131070]
    value  = float32(s) * float32(sigma / 37837.227)                  one IEEE rounding

The sum of four uniform 16-bit fields (Irwin-Hall) has standard deviation 65536 / sqrt(3) =
37837.227 and is close to normal (it ends at 3.46 sigma).  Integer arithmetic and a single float32
multiplication are bit-identical in numpy and in torch on any device, so a rank can generate
exactly its own rows or columns on its GPU and the CPU checker the whole tensor.

`index` is the element's position in the WHOLE (unsliced) row-major tensor.
"""
import numpy as np

MASK64 = (1 << 64) - 1
_STD = 37837.227

# tensor ids
X, W_GATE, W_UP, W_DOWN, W_NORM = 0, 1, 2, 3, 4


def _key(seed, tensor, layer):
    """A 64-bit stream key: distinct streams for every (seed, tensor, layer)."""
    k = (seed * 0x9E3779B97F4A7C15 + tensor * 0xD1B54A32D192ED03 + layer * 0x8CB92BA72F3D8DD7 + 0x2545F4914F6CDD1D) & MASK64
    k ^= k >> 29
    k = (k * 0xBF58476D1CE4E5B9) & MASK64
    return k ^ (k >> 32)


def _scale(sigma):
    return np.float32(np.float32(sigma) / np.float32(_STD))


def values_numpy(seed, tensor, layer, index, sigma):
    """index: integer array (any shape) of whole-tensor element positions -> float32 array."""
    with np.errstate(over="ignore"):
        z = index.astype(np.uint64) + np.uint64(_key(seed, tensor, layer))
        z += np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
    m = np.uint64(0xFFFF)
    s = ((z & m) + ((z >> np.uint64(16)) & m) + ((z >> np.uint64(32)) & m) + (z >> np.uint64(48))).astype(np.int64) - 131070
    return s.astype(np.float32) * _scale(sigma)


def _signed(v):
    v &= MASK64
    return v - (1 << 64) if v >= (1 << 63) else v


def values_torch(seed, tensor, layer, index, sigma):
    """The same on a torch int64 tensor of positions (any device): two's-complement int64 arithmetic
    wraps like uint64, logical right shifts are an arithmetic shift plus a mask."""
    import torch

    def lsr(v, s):
        return (v >> s) & ((1 << (64 - s)) - 1)

    z = index + _signed(_key(seed, tensor, layer))
    z = z + _signed(0x9E3779B97F4A7C15)
    z = (z ^ lsr(z, 30)) * _signed(0xBF58476D1CE4E5B9)
    z = (z ^ lsr(z, 27)) * _signed(0x94D049BB133111EB)
    z = z ^ lsr(z, 31)
    s = (z & 0xFFFF) + (lsr(z, 16) & 0xFFFF) + (lsr(z, 32) & 0xFFFF) + lsr(z, 48) - 131070
    return s.to(torch.float32) * float(_scale(sigma))


def matrix_numpy(seed, tensor, layer, rows, cols, sigma, row_block=2048):
    """The whole [rows, cols] tensor as float32 (generated in row blocks to bound the temporaries)."""
    out = np.empty((rows, cols), np.float32)
    c = np.arange(cols, dtype=np.uint64)[None, :]
    for r0 in range(0, rows, row_block):
        r = np.arange(r0, min(rows, r0 + row_block), dtype=np.uint64)[:, None]
        out[r0:r0 + r.shape[0]] = values_numpy(seed, tensor, layer, r * np.uint64(cols) + c, sigma)
    return out


def matrix_torch(seed, tensor, layer, rows, cols, sigma, device, row_off=0, nrows=None, col_off=0, ncols=None,
                 row_block=4096):
    """Rows [row_off, row_off + nrows) x columns [col_off, col_off + ncols) of the whole [rows, cols]
    tensor, on `device`, as float32."""
    import torch
    nrows = rows - row_off if nrows is None else nrows
    ncols = cols - col_off if ncols is None else ncols
    out = torch.empty((nrows, ncols), dtype=torch.float32, device=device)
    c = torch.arange(col_off, col_off + ncols, dtype=torch.int64, device=device)[None, :]
    for r0 in range(0, nrows, row_block):
        n = min(row_block, nrows - r0)
        r = torch.arange(row_off + r0, row_off + r0 + n, dtype=torch.int64, device=device)[:, None]
        out[r0:r0 + n] = values_torch(seed, tensor, layer, r * cols + c, sigma)
    return out


def stack_layer_torch(seed, layer, hidden, inter, tp, rank, device, with_norm=True):
    """Rank `rank` of `tp`'s operands of layer `layer` of the synthetic stack, quantized on the device
    with the library's quantizer (the reference's format, byte for byte): gate rows and up rows
    [rank*I/tp, (rank+1)*I/tp), down columns likewise (a column slice on a group boundary quantizes to
    exactly the bytes and scales the whole tensor's quantization has there).  Returns a DenseMlp."""
    import torch
    from .ops import DenseMlp, quantize_int4
    per = inter // tp
    if per * tp != inter or per % 128:
        raise ValueError("the split must fall on a 128-group boundary")
    gp, gs = quantize_int4(matrix_torch(seed, W_GATE, layer, inter, hidden, 0.02, device, row_off=rank * per, nrows=per))
    up, us = quantize_int4(matrix_torch(seed, W_UP, layer, inter, hidden, 0.02, device, row_off=rank * per, nrows=per))
    dp, ds = quantize_int4(matrix_torch(seed, W_DOWN, layer, hidden, inter, 0.02, device, col_off=rank * per, ncols=per).contiguous())
    norm = None
    if with_norm:
        norm = matrix_torch(seed, W_NORM, layer, 1, hidden, 0.1, device).reshape(hidden).to(torch.bfloat16)
    return DenseMlp(torch.cat([gp, up]), torch.cat([gs, us]), dp, ds, post_norm_w=norm)


def stack_input_torch(seed, tokens, hidden, device):
    import torch
    return matrix_torch(seed, X, 0, tokens, hidden, 1.0, device).to(torch.bfloat16)
