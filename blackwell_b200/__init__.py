"""blackwell_b200 -- the INT4 block-16 GEMV decode path as sm_100a CUDA kernels.

The product is the shared library ``blackwell_b200/lib/libblackwell_kernels.so``
(C ABI in ``include/blackwell_b200.h``; the reference's C++ symbols in
``include/blackwell_b200_dropin.hpp``).  This package only loads it and offers
thin tensor-level wrappers with the reference's function names:

    from blackwell_b200 import kernels
    kernels.gemv_int4_batched(y, x_packed, x_scale, W_packed, W_scale, K, N, M)

There is no CPU or PyTorch fallback: importing ``kernels`` without the built
library raises.
"""
__all__ = ["kernels", "synth", "shapes"]
