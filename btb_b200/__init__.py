"""btb_b200 - a B200-native (sm_100a) decode hot path behind btb's card-kernel seam.

``capi``      ctypes binding of the C-ABI in include/btb_b200.h (libbtb_b200.so, built by ``btb_b200.build``)
``launcher``  a drop-in for btb's ``Launcher`` protocol: the reference's kernel names on this library
``engine``    the card graph's step (embed -> layers -> head -> pick -> publish) and greedy loop
``pack12`` / ``mxfp4`` / ``fp8``  host-side codecs of the weight formats the kernels read as stored
"""

__all__ = ["capi", "launcher", "engine", "pack12"]
