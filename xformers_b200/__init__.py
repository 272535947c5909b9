"""B200-native (sm_100a) attention forward behind the xFormers fmha API.

``import xformers_b200.ops as xops`` gives ``xops.memory_efficient_attention_forward``,
``xops.fmha.attn_bias``, ``xops.fmha.merge_attentions`` with hand-written CUDA
kernels from ``csrc/`` (libxfb200.so, C ABI in ``include/xfb200.h``).
"""

__version__ = "0.1.0"
