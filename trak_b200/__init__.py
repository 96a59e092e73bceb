"""trak_b200: B200 (sm_100a) kernels for TRAK's JL projection and after-kernel scoring.

The CUDA code sits behind the C ABI of ``include/trak_b200.h``
(``libtrakb200.so``); this package mirrors the reference's Python surface for
those paths: the ``fast_jl`` entry points, the projector classes and a score
computer.
"""
__version__ = "0.1.0"
