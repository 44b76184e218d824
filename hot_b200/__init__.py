"""hot_b200: the HOT (Hadamard-based Optimized Training) linear-layer backward on B200.

The arithmetic lives in hand-written sm_100a CUDA behind a C ABI (``include/hot_b200.h``,
built into ``hot_b200/lib/libhot_b200.so`` by ``python -m hot_b200.build``); this package is
the host-side mirror of the reference's operator interface on top of it.
"""
__version__ = "0.1.0"
