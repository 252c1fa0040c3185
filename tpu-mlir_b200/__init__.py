"""B200 (sm_100a) backend for tpu-mlir's quantized-inference hot path.

The product is ``libb200q.so`` (hand-written CUDA kernels behind a C ABI, ``include/b200q.h``); this
package is the thin Python mirror of the reference's operator and module interfaces on top of it.
There is no CPU fallback: without the built library or without a CUDA device the ops raise.
"""
__version__ = "0.1"
