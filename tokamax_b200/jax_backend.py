"""tokamax backend ``implementation="cuda_sm100"``: the B200 splash kernels behind ``tokamax.Op``.

NOT RUN where this package was developed: JAX and tokamax are not installed there, so this module
has only been read against the interfaces it implements.  It imports ``jax`` and ``tokamax`` at the
top and therefore fails with ``ImportError`` where they are missing; nothing else in the package
imports it.

What it does, with the reference interface each piece stands in for:

* ``CudaSm100SplashAttention`` subclasses ``DotProductAttention`` and overrides ``_fwd`` with the
  signature of ``tokamax/_src/ops/attention/base.py:564-584``; it plays the role of
  ``PallasMosaicTpuFlashAttention`` (``pallas_mosaic_tpu.py:62-173``): same input checks
  (``pallas_mosaic_tpu_common.py:30-62``), same mask mapping (``:64-117``: boolean mask, causal, or
  full), residuals ``(max_logits, logsumexp)`` shaped ``[*B, H, T]`` (``pallas_mosaic_tpu.py:154-166``).
* ``CudaSm100SplashAttentionVjp`` overrides ``DotProductAttentionVjp._fwd`` (``base.py:813-843``)
  the way ``PallasMosaicTpuFlashAttentionVjp`` does (``pallas_mosaic_tpu_vjp.py:64-244``).
* ``register()`` registers the two XLA FFI targets of ``csrc/splash_xla_ffi.cc`` and adds the
  backend to ``tokamax._src.ops.attention.api.IMPLEMENTATIONS`` (``api.py:37-80``), after which
  ``tokamax.dot_product_attention(..., implementation="cuda_sm100")`` dispatches to it and falls
  through to the next implementation on ``NotImplementedError`` (``api.py:187-192``).

Differences from the TPU adapter: ``[*B, T, H, D]`` tensors are passed to the kernels as they are
(handler attribute ``layout=1``; the four transposes of ``pallas_mosaic_tpu.py:121-124`` do not
happen), the softmax scale is applied in fp32 inside the kernel instead of ``q *= logits_scale``,
and the batch is a grid dimension instead of ``jax.vmap``.  Masks must be concrete (host) values:
the schedules are built on the host and enter the computation as constants.
"""

from __future__ import annotations

import dataclasses
from typing import Any, ClassVar

try:
  import jax
  import jax.numpy as jnp
except ImportError as e:  # pragma: no cover
  raise ImportError("tokamax_b200.jax_backend needs jax (and tokamax); neither is a dependency of the rest of "
                    "this package") from e
import numpy as np
from tokamax._src.ops import op as op_lib  # pylint: disable=g-import-not-at-top
from tokamax._src.ops.attention import api as attention_api
from tokamax._src.ops.attention import base as attention_base

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import xla_ffi

_registered = False

# Autotuning-cache entries for this backend in the reference's format
# (tokamax/_src/autotuning/cache.py:72-112: <cache dir>/<device kind>/<op name>.json, bound
# arguments -> config -> timings) ship in tokamax_b200/data/autotuning/nvidia_b200/; pass that
# directory to tokamax's AutotuningCache(paths=[...]) to have them picked up.
AUTOTUNING_CACHE_DIR = "data/autotuning"


@dataclasses.dataclass(frozen=True)
class Config:
  """The backend's only configuration: the MaskInfo block size (the MMA tile is fixed at 128 x 128)."""
  block_q: int = 128
  block_kv: int = 128


def _register_ffi_targets() -> None:
  global _registered
  if _registered:
    return
  lib = _native.lib()
  if not lib.splash_xla_ffi_compiled():
    raise RuntimeError(
        "libsplash_b200.so was built without the XLA FFI handlers; rebuild it with jaxlib's include directory "
        "(jaxlib/include, which holds xla/ffi/api/ffi.h) on the compiler's include path")
  for which, target in xla_ffi.TARGET_NAMES.items():
    handler = getattr(lib, xla_ffi.HANDLER_SYMBOLS[which])
    jax.ffi.register_ffi_target(target, jax.ffi.pycapsule(handler), platform="CUDA")
  _registered = True


def _check_inputs(q, k, v, *, bias, logits_dtype, dropout_mask, dropout_rate, paging_info, mask, q_indices, k_indices,
                  normalize_output):
  """pallas_mosaic_tpu_common.py:30-62, plus what the B200 kernels add or lack."""
  if any(x.dtype != jnp.bfloat16 for x in (q, k, v)):
    raise NotImplementedError("Only bfloat16 inputs are built on B200.")
  if bias is not None:
    raise NotImplementedError("Bias is not supported.")
  if logits_dtype != jnp.float32:
    raise NotImplementedError("`logits_dtype` must be float32.")
  if dropout_mask is not None or dropout_rate != 0.0:
    raise NotImplementedError("dropout is not supported.")
  if paging_info is not None:
    raise NotImplementedError("Paged attention not supported.")
  if q_indices is not None or k_indices is not None:
    raise NotImplementedError("q_indices / k_indices are not supported.")
  if not normalize_output:
    raise NotImplementedError("`normalize_output=False` is not supported.")
  for name in ("q_start", "q_end", "k_start", "k_end"):
    if getattr(mask, name) is not None:
      raise NotImplementedError(f"mask.{name} is not supported.")
  if q.shape[-1] > 256 or v.shape[-1] > 256 or q.shape[-1] % 8 or v.shape[-1] % 8:
    raise NotImplementedError("head dims must be multiples of 8, at most 256")
  if q.shape[-3] % 128 or k.shape[-3] % 128:
    raise NotImplementedError("sequence lengths must be multiples of 128")


def _splash_kernel(mask, q_len: int, kv_len: int, soft_cap):
  """pallas_mosaic_tpu_common.py:64-117 with host-side masks."""
  config = dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=soft_cap)
  if mask.bool_mask is not None:
    dense = mask.as_array(q_len, kv_len)
    if isinstance(dense, jax.core.Tracer):
      raise NotImplementedError("a traced boolean mask cannot be turned into host-side schedules")
    dense = np.asarray(dense)
    dense = dense.reshape((-1,) + dense.shape[-2:])
    if dense.shape[0] != 1:
      raise NotImplementedError("only a [T, S] mask shared by batch and heads is supported")
    splash_mask = mask_lib.NumpyMask(np.ascontiguousarray(dense[0], dtype=np.bool_))
  elif mask.is_causal:
    splash_mask = mask_lib.CausalMask((q_len, kv_len))
  else:
    splash_mask = mask_lib.FullMask((q_len, kv_len))
  return splash.make_splash_mha(splash_mask, q_seq_shards=1, config=config, save_residuals=True,
                                mask_value=float(np.finfo(np.float32).min), downcast_smem_data=False)


def _as_4d(x):
  return jax.lax.collapse(jax.lax.broadcast_to_rank(x, 4), 0, -3)


def _operands(plan, runtime: dict[str, Any]):
  out = []
  for name, const in plan["operands"]:
    if const is not None:
      out.append(jnp.asarray(const))
    elif runtime.get(name) is not None:
      out.append(runtime[name])
    else:  # an optional runtime operand that is absent: zero elements, read as NULL by the handler
      out.append(jnp.zeros((0,), jnp.float32 if name in ("sinks", "max_logit_value") else jnp.int32))
  return out


@dataclasses.dataclass(frozen=True)
class CudaSm100SplashAttentionVjp(attention_base.DotProductAttentionVjp):
  """dq / dk / dv through ``splash_bwd`` (fused form)."""

  supports_symbolic_shapes: ClassVar[bool] = False

  def _fwd(self, residuals, out, dout, q, k, v, *, precision, logits_dtype, logits_scale, bias, logits_soft_cap, mask,
           dropout_mask, dropout_rate, paging_info, q_indices, k_indices, normalize_output, return_residuals, config):
    del precision, config
    if return_residuals:
      raise NotImplementedError("`return_residuals` not supported.")
    _check_inputs(q, k, v, bias=bias, logits_dtype=logits_dtype, dropout_mask=dropout_mask, dropout_rate=dropout_rate,
                  paging_info=paging_info, mask=mask, q_indices=q_indices, k_indices=k_indices,
                  normalize_output=normalize_output)
    _register_ffi_targets()
    _, logsumexp = residuals
    shapes = (q.shape, k.shape, v.shape)
    q4, k4, v4, o4, do4 = map(_as_4d, (q, k, v, out, dout))
    b, t, h, _ = q4.shape
    kernel = _splash_kernel(mask, t, k4.shape[1], logits_soft_cap)
    plan = xla_ffi.call_plan(kernel, xla_ffi.BWD, scale=float(logits_scale), layout=xla_ffi.LAYOUT_BSHD)
    ws_bytes = int(_native.lib().splash_bwd_fused_workspace_bytes(b, h, t))
    results = (jax.ShapeDtypeStruct(q4.shape, q4.dtype), jax.ShapeDtypeStruct(k4.shape, k4.dtype),
               jax.ShapeDtypeStruct(v4.shape, v4.dtype), jax.ShapeDtypeStruct((ws_bytes,), jnp.uint8),
               jax.ShapeDtypeStruct((4,), jnp.uint32))
    runtime = dict(q=q4, k=k4, v=v4, o=o4, d_o=do4, logsumexp=logsumexp.reshape(b, h, t))
    dq, dk, dv, _, _ = jax.ffi.ffi_call(plan["target"], results)(*_operands(plan, runtime), **plan["attrs"])
    grads = {"q": dq.reshape(shapes[0]), "k": dk.reshape(shapes[1]), "v": dv.reshape(shapes[2])}
    return grads, None


@dataclasses.dataclass(frozen=True)
class CudaSm100SplashAttention(attention_base.DotProductAttention):
  """Splash attention on B200 through the XLA custom call."""

  config_cls: ClassVar[type[Config]] = Config
  supports_symbolic_shapes: ClassVar[bool] = False

  def __post_init__(self):
    if self.vjp is None:
      object.__setattr__(self, "vjp", CudaSm100SplashAttentionVjp())

  def _fwd(self, q, k, v, *, precision, logits_dtype, logits_scale, bias, logits_soft_cap, mask, dropout_mask,
           dropout_rate, paging_info, q_indices, k_indices, normalize_output, return_residuals, config):
    del precision, config
    _check_inputs(q, k, v, bias=bias, logits_dtype=logits_dtype, dropout_mask=dropout_mask, dropout_rate=dropout_rate,
                  paging_info=paging_info, mask=mask, q_indices=q_indices, k_indices=k_indices,
                  normalize_output=normalize_output)
    _register_ffi_targets()
    orig_q_shape = q.shape
    q4, k4, v4 = map(_as_4d, (q, k, v))
    b, t, h, _ = q4.shape
    if h % k4.shape[2]:
      raise ValueError(f"num_q_heads={h} must be divisible by num_kv_heads={k4.shape[2]}")
    kernel = _splash_kernel(mask, t, k4.shape[1], logits_soft_cap)
    plan = xla_ffi.call_plan(kernel, xla_ffi.FWD, scale=float(logits_scale), layout=xla_ffi.LAYOUT_BSHD)
    results = (jax.ShapeDtypeStruct(q4.shape[:-1] + (v4.shape[-1],), q4.dtype), jax.ShapeDtypeStruct((b, h, t), jnp.float32),
               jax.ShapeDtypeStruct((b, h, t), jnp.float32), jax.ShapeDtypeStruct((4,), jnp.uint32))
    out, logsumexp, max_logits, _ = jax.ffi.ffi_call(plan["target"], results)(
        *_operands(plan, dict(q=q4, k=k4, v=v4)), **plan["attrs"])
    out = out.reshape(*orig_q_shape[:-1], out.shape[-1])
    residuals = None
    if return_residuals:
      shape = (*orig_q_shape[:-3], orig_q_shape[-2], orig_q_shape[-3])  # [*B, H, T]
      residuals = (max_logits.reshape(shape), logsumexp.reshape(shape))
    return out, residuals

  def _get_heuristics_config(self, ba: op_lib.BoundArguments):
    return Config()  # the MMA tile is fixed at 128 x 128; there is nothing to tune per call

  def _get_autotuning_configs(self, ba: op_lib.BoundArguments) -> set[Config]:
    return {Config()}

  def supported_on(self, device: jax.Device) -> bool:
    if device.platform != "gpu":
      return False
    capability = getattr(device, "compute_capability", "")
    return str(capability).startswith("10")


def register(name: str = "cuda_sm100") -> None:
  """Adds the backend to tokamax's implementation table (api.py:37-80 builds an immutabledict, so
  the table is replaced, not mutated)."""
  impls = dict(attention_api.IMPLEMENTATIONS)
  impls[name] = CudaSm100SplashAttention()
  attention_api.IMPLEMENTATIONS = type(attention_api.IMPLEMENTATIONS)(impls)
