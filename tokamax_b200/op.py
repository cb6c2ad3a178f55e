"""``dot_product_attention(..., implementation="cuda_sm100")`` — the Op-level entry point.

Torch counterpart of the reference's attention API
(``tokamax/_src/ops/attention/api.py:83-192``) and of the adapter that puts splash attention
behind it (``tokamax/_src/ops/attention/pallas_mosaic_tpu.py:62-231``,
``pallas_mosaic_tpu_common.py:30-117``): same argument names and layout
(``query [*B, T, N, H]``, ``key / value [*B, S, K, H]``), the same "first implementation that does
not raise NotImplementedError wins" dispatch, and the same list of features the splash backend
rejects (bias, dropout, paging, per-example sequence lengths).

Differences that matter on B200: the softmax scale is applied in fp32 inside the kernel instead
of scaling q in bf16, and the ``[B, T, N, H]`` tensors are read and written in place through
strides — the reference's four layout transposes (``pallas_mosaic_tpu.py:121-124``) do not exist.
"""

from __future__ import annotations

import dataclasses
import functools
from typing import Any, Callable, Sequence

import numpy as np
import torch

from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

AUTO = "auto"
_LIVE_KERNELS: list = []


@functools.lru_cache(maxsize=32)
def _kernel_for(kind: str, t: int, s: int, window: tuple | None, dense_key: bytes | None,
                soft_cap: float | None = None):
  if kind == "dense":
    dense = np.frombuffer(dense_key, dtype=np.bool_).reshape(t, s)
    mask = mask_lib.NumpyMask(dense.copy())
  elif kind == "full":
    mask = mask_lib.FullMask((t, s))
  elif kind == "causal":
    mask = mask_lib.CausalMask((t, s))
  elif kind == "local":
    mask = mask_lib.LocalMask((t, s), window, 0)
  else:
    raise ValueError(kind)
  config = None
  if soft_cap is not None:
    config = dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=soft_cap)
  kernel = splash.make_splash_mha(mask, q_seq_shards=1, save_residuals=True, config=config,
                                  mask_value=float(np.finfo(np.float32).min), downcast_smem_data=False)
  _LIVE_KERNELS.append(kernel)
  del _LIVE_KERNELS[:-64]  # the cache above holds 32; keep the list bounded the same way
  return kernel


class CudaSm100SplashAttention:
  """Splash attention on B200 behind the Op interface (forward and, through autograd, vjp)."""

  def supported_on(self, device: torch.device) -> bool:
    return device.type == "cuda" and torch.cuda.get_device_capability(device)[0] == 10

  def __call__(self, query, key, value, *, bias=None, mask=None, is_causal=False, local_window_size=None,
               logits_scale: float | str = AUTO, logits_soft_cap=None, dropout_rate: float = 0.0,
               query_seq_lengths=None, key_value_seq_lengths=None, return_residuals: bool = False,
               precision=None, q_sharding=None):
    if bias is not None:
      raise NotImplementedError("Bias is not supported.")
    if dropout_rate != 0.0:
      raise NotImplementedError("dropout is not supported.")
    if query_seq_lengths is not None or key_value_seq_lengths is not None:
      raise NotImplementedError("per-example sequence lengths (k-ranges) are not supported.")
    if q_sharding is not None:
      raise NotImplementedError("q_sharding is a JAX construct; use tokamax_b200.ulysses")
    if query.dtype != torch.bfloat16 or key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
      raise NotImplementedError(f"only bfloat16 is built on B200, got {query.dtype}")
    if query.dim() < 3 or key.dim() != query.dim() or value.dim() != query.dim():
      raise ValueError(f"expected [*B, T, N, H] tensors, got {tuple(query.shape)}, {tuple(key.shape)}")
    if not self.supported_on(query.device):
      raise NotImplementedError(f"cuda_sm100 needs a B200-class CUDA device, got {query.device}")
    *batch, t, n, h = query.shape
    s, k_heads = key.shape[-3], key.shape[-2]
    if list(key.shape[:-3]) != batch or list(value.shape[:-3]) != batch:
      raise ValueError("batch dimensions of query, key and value differ")
    if h > 256 or value.shape[-1] > 256:
      raise NotImplementedError(f"head dims above 256 are not built on B200, got {h} / {value.shape[-1]}")
    if t % 128 or s % 128:
      raise NotImplementedError("sequence lengths must be multiples of 128")
    scale = h ** -0.5 if logits_scale == AUTO else float(logits_scale)
    cap = None if logits_soft_cap is None else float(logits_soft_cap)

    if isinstance(mask, torch.Tensor) and mask.is_cuda:
      # A mask that is data on the device takes the dynamic path, as the reference's adapter does
      # for array masks (pallas_mosaic_tpu_common.py:96-102): tile states and schedules are built
      # on the device, nothing is copied to the host.
      m = mask.to(torch.bool)
      while m.dim() > 2 and m.shape[0] == 1:
        m = m[0]
      if m.dim() != 2:
        raise NotImplementedError("only a [T, S] mask shared by batch and heads is supported")
      m = m.expand(t, s)
      if is_causal or local_window_size is not None:
        rel = torch.arange(s, device=m.device)[None, :] - torch.arange(t, device=m.device)[:, None]  # k - q
        if is_causal:
          m = m & (rel <= 0)
        if local_window_size is not None:
          w = (local_window_size, local_window_size) if isinstance(local_window_size, int) else tuple(local_window_size)
          if w[0] is not None:
            m = m & (rel >= -w[0])
          if w[1] is not None:
            m = m & (rel <= w[1])
      config = None
      if cap is not None:
        config = dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=cap)
      kernel = splash.make_dynamic_splash_mha(m.contiguous(), save_residuals=True, config=config,
                                              mask_value=float(np.finfo(np.float32).min), downcast_smem_data=False)
    elif mask is not None:
      m = np.asarray(mask.detach().cpu() if hasattr(mask, "detach") else mask).astype(np.bool_)
      while m.ndim > 2 and m.shape[0] == 1:
        m = m[0]
      if m.ndim != 2:
        raise NotImplementedError("only a [T, S] mask shared by batch and heads is supported")
      m = np.broadcast_to(m, (t, s))
      if is_causal:
        m = m & mask_lib.make_causal_mask((t, s))
      if local_window_size is not None:
        w = (local_window_size, local_window_size) if isinstance(local_window_size, int) else tuple(local_window_size)
        m = m & mask_lib.make_local_attention_mask((t, s), w)
      kernel = _kernel_for("dense", t, s, None, np.ascontiguousarray(m).tobytes(), cap)
    elif local_window_size is not None:
      w = (local_window_size, local_window_size) if isinstance(local_window_size, int) else tuple(local_window_size)
      if is_causal:
        w = (w[0], min(w[1], 0) if w[1] is not None else 0)
      kernel = _kernel_for("local", t, s, w, None, cap)
    elif is_causal:
      kernel = _kernel_for("causal", t, s, None, None, cap)
    else:
      kernel = _kernel_for("full", t, s, None, None, cap)

    def bhtd(x):  # [*B, L, N, H] -> [B', N, L, H] view, no copy for a single batch axis
      x = x.reshape((-1,) + tuple(x.shape[-3:])) if len(batch) != 1 else x
      return x.permute(0, 2, 1, 3)

    out, res = kernel(bhtd(query), bhtd(key), bhtd(value), logits_scale=scale)
    out = out.permute(0, 2, 1, 3).reshape(tuple(batch) + (t, n, value.shape[-1]))
    if return_residuals:
      shape = tuple(batch) + (n, t)
      return out, (res["max_logits"].reshape(shape), res["logsumexp"].reshape(shape))
    return out


def check_errors() -> None:
  """Raises if any kernel object this module has built for static masks reported a device-side
  fault (a bounded wait that ran out); see ``SplashAttentionKernel.check_errors``.  Kernel objects
  for masks that are device tensors are built per call and are not tracked here."""
  # functools.lru_cache keeps no public view of its values: the kernels register themselves
  for kernel in list(_LIVE_KERNELS):
    kernel.check_errors()


IMPLEMENTATIONS: dict[str, Callable[..., Any]] = {"cuda_sm100": CudaSm100SplashAttention()}
_DEFAULT_IMPLEMENTATIONS = ("cuda_sm100",)


def dot_product_attention(query, key, value, bias=None, mask=None, *, scale: float | None = None,
                          is_causal: bool = False, query_seq_lengths=None, key_value_seq_lengths=None,
                          local_window_size: int | tuple[int, int] | None = None, logits_soft_cap=None,
                          precision=None, implementation: str | Sequence[str] | None = None, q_sharding=None):
  """Scaled dot-product attention, ``query [*B, T, N, H]``; dispatches over ``implementation``."""
  if implementation is None:
    implementation = _DEFAULT_IMPLEMENTATIONS
  elif isinstance(implementation, str):
    implementation = (implementation,)
  elif not implementation:
    raise ValueError("`implementation` must not be an empty sequence.")
  errors = []
  for impl in implementation:
    if isinstance(impl, str):
      if impl not in IMPLEMENTATIONS:
        raise ValueError(f"Unknown implementation: {impl}")
      impl = IMPLEMENTATIONS[impl]
    try:
      return impl(query, key, value, bias=bias, mask=mask, is_causal=is_causal,
                  local_window_size=local_window_size, logits_scale=AUTO if scale is None else scale,
                  logits_soft_cap=logits_soft_cap, query_seq_lengths=query_seq_lengths,
                  key_value_seq_lengths=key_value_seq_lengths, precision=precision, q_sharding=q_sharding)
    except NotImplementedError as e:
      if len(implementation) == 1:
        raise
      errors.append(e)
  raise ExceptionGroup("all implementations failed", errors)
