"""tokamax_b200 — splash attention for NVIDIA B200 (sm_100a).

A from-scratch implementation of one hot path of tokamax: the host-side ``MaskInfo`` builder,
the splash-attention forward kernel, the dq / dkv backward kernels and a context-parallel
(Ulysses) wrapper, behind the reference's Python names.  Device work is hand-written CUDA
(tcgen05 MMAs, TMEM accumulators, TMA) reached through the C ABI in ``include/splash_b200.h``.
"""

from tokamax_b200 import base
from tokamax_b200 import splash_attention_mask
from tokamax_b200 import splash_attention_mask_info
from tokamax_b200.base import DEFAULT_MASK_VALUE, SegmentIds
from tokamax_b200.splash_attention_mask import (
    CausalMask,
    ChunkedCausalMask,
    FullMask,
    LocalMask,
    LogicalAnd,
    LogicalOr,
    Mask,
    NumpyMask,
    make_causal_mask,
    make_chunk_attention_mask,
    make_local_attention_mask,
    make_random_mask,
)
from tokamax_b200.splash_attention_mask_info import MaskInfo, find_bounds, process_mask, process_mask_dkv

__all__ = [
    "base", "splash_attention_mask", "splash_attention_mask_info",
    "DEFAULT_MASK_VALUE", "SegmentIds", "MaskInfo", "find_bounds", "process_mask", "process_mask_dkv",
    "Mask", "CausalMask", "ChunkedCausalMask", "LocalMask", "FullMask", "NumpyMask", "LogicalAnd",
    "LogicalOr", "make_causal_mask", "make_local_attention_mask", "make_chunk_attention_mask",
    "make_random_mask",
]


def __getattr__(name):
  # The kernel module imports torch; keep `import tokamax_b200` light for table-only users.
  if name in ("splash_attention_kernel", "ulysses", "ring_attention", "op", "fp8"):
    import importlib

    return importlib.import_module(f"tokamax_b200.{name}")
  if name in ("SplashConfig", "QKVLayout", "SplashAttentionKernel", "make_splash_mha", "make_splash_mqa",
              "make_splash_mha_single_device", "make_splash_mqa_single_device",
              "make_dynamic_splash_mha", "make_dynamic_splash_mqa"):
    from tokamax_b200 import splash_attention_kernel as _k

    return getattr(_k, name)
  raise AttributeError(name)
