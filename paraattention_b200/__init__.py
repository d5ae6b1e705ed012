"""B200-native context-parallel attention engine with the ParaAttention API surface.

The compute path is the CUDA library ``libpa_b200.so`` (hand-written sm_100a kernels behind a
C ABI, see ``include/pa_b200.h``); this package is the host-side mirror of the reference's
Python interface for that path. There is no CPU or PyTorch fallback.
"""

__version__ = "0.1.0"
