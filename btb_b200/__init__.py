"""btb_b200 - a B200-native (sm_100a) decode hot path behind btb's card-kernel seam.

``capi``      ctypes binding of the C-ABI in include/btb_b200.h (libbtb_b200.so, built by ``btb_b200.build``)
``launcher``  a drop-in for btb's ``Launcher`` protocol: the reference's kernel names on this library
``engine``    the card graph's step (embed -> layers -> head -> pick -> publish), greedy loop and prefill
``moe``       the MoE decoder: router, picked experts over MXFP4 / FP8 / bf16 as stored, ordered sum
``batch``     small-batch decode: B sequences through one pass of B rows; btb's rows layout (forks of a shared prefix)
``session``   btb's session surface over an engine: feed / mark / rewind / crop / generate
``paged``     the paged cache with a shared-prefix tree
``parallel``  one dense model tensor-parallel over the GPUs of a box; ``exchange`` its peer-mapped memory
``draft``     n-gram drafting and the speculative greedy loop; ``sampling`` the sampled pick's host side
``pack12``    btb's 12-bit lossless bf16 store, encoded on the card
"""

__all__ = ["capi", "launcher", "engine", "moe", "batch", "session", "paged", "parallel", "exchange", "draft", "sampling", "pack12"]
