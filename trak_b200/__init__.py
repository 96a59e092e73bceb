"""trak_b200: B200 (sm_100a) kernels for TRAK's JL projection and after-kernel scoring.

The CUDA code sits behind the C ABI of ``include/trak_b200.h``
(``libtrakb200.so``); this package mirrors the reference's Python surface for
those paths: the ``fast_jl`` entry points, the projector classes and a score
computer.
"""
__version__ = "0.1.0"


def install_fast_jl_shim() -> None:
    """Registers ``trak_b200.fast_jl`` under the module name ``fast_jl``, so that an unmodified ``trak``
    (``import fast_jl`` in trak/projectors.py:373 and trak/traker.py:254-262) picks up the sm_100a kernels."""
    import sys
    from . import fast_jl
    sys.modules["fast_jl"] = fast_jl
