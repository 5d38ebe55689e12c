"""B200-native weight-only INT4 dense-FFN decode path (drop-in for the reference's
``forward_mlp`` / ``gemm_int4_bf16`` / ``allreduce_sum`` / ``engine_load_quantized_ffn`` path).

The product is ``libffn_int4.so`` (CUDA C++ for sm_100a behind the C ABI of
``include/ffn_int4.h``).  This package is the thin host-side mirror used by the tests and the
benchmark: it loads the library with ctypes and passes raw device pointers; PyTorch only owns
device memory and streams.  There is no CPU fallback - importing :mod:`.lib` without the built
library raises.
"""
from .lib import load, LibraryMissing, check  # noqa: F401
