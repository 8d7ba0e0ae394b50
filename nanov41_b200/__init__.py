"""B200-native (sm_100a) MoE expert path with the call signatures of nanov41's
``fast_moe`` / ``moe_triton`` / ``triton_grouped_moe`` modules.

Everything numeric runs in the hand-written CUDA library ``csrc/libnanov41_b200.so`` through
its C ABI (``include/nanov41_b200.h``); PyTorch only owns device memory and streams.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
