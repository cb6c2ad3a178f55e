"""Host side of the XLA custom-call adapter (``csrc/splash_xla_ffi.cc``), free of any JAX import.

The adapter's handlers take their operands, results and attributes in one fixed order, which the
library reports through ``splash_xla_ffi_signature``.  This module parses that report, maps every
name onto the field of ``SplashFwdArgs`` / ``SplashBwdArgs`` it fills (so a test can check that the
two stay in step), and builds the host-side pieces of a call — the schedules as numpy arrays and
the attribute dictionary — from a ``SplashAttentionKernel``.  ``tokamax_b200/jax_backend.py`` turns
those into ``jax.ffi.ffi_call`` arguments.
"""

from __future__ import annotations

import numpy as np

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_mask_info as mask_info_lib

FWD, BWD = 0, 1
TARGET_NAMES = {FWD: "splash_b200_fwd", BWD: "splash_b200_bwd"}
HANDLER_SYMBOLS = {FWD: "SplashFwd", BWD: "SplashBwd"}
LAYOUT_BHSD, LAYOUT_BSHD = 0, 1
_NP_KIND = {"s32": np.int32, "s8": np.int8, "u8": np.uint8, "u32": np.uint32, "f32": np.float32}


def signature(which: int) -> dict[str, list[tuple[str, str]]]:
  """``{"operands": [(name, kind), ...], "results": [...], "attrs": [(name, c_type), ...]}``."""
  text = _native.lib().splash_xla_ffi_signature(which).decode()
  out = {}
  for part in text.split(";"):
    if not part:
      continue
    key, _, items = part.partition("=")
    out[key] = [tuple(item.split(":")) for item in items.split(",") if item]
  return out


def field_path(name: str, which: int) -> str | None:
  """The ``SplashFwdArgs`` / ``SplashBwdArgs`` field a handler argument fills (dotted path), or
  None for ``layout``, which only says how the rank-4 buffers are to be viewed."""
  if name == "layout":
    return None
  if name in ("sched_block_q", "sched_block_kv"):
    leaf = name[len("sched_"):]
    return f"sched.{leaf}" if which == FWD else f"sched_dq.{leaf}+sched_dkv.{leaf}"
  for prefix, struct in (("sched_", "sched"), ("dq_", "sched_dq"), ("dkv_", "sched_dkv")):
    if name.startswith(prefix) and (which == FWD) == (prefix == "sched_"):
      return f"{struct}.{name[len(prefix):]}"
  if name.startswith("mask_") and name != "mask_value":
    return f"mask_fn.{name[len('mask_'):]}"
  return name


def host_schedules(kernel) -> dict[str, dict[str, np.ndarray | None]]:
  """The three kernel schedules of ``kernel`` as host arrays: ``{"fwd" | "dq" | "dkv": {"row_ptr",
  "entries", "row_order", "partial_mask_blocks"}}`` (what ``_DeviceTables`` uploads for torch)."""
  from tokamax_b200 import splash_attention_kernel as splash  # pylint: disable=g-import-not-at-top

  cfg = kernel.config
  fwd, dkv = kernel.fwd_mask_info, kernel.dkv_mask_info
  q_len, kv_len = kernel.mask_shape
  state, pid = mask_info_lib.block_grids(fwd, q_len // cfg.block_q, kv_len // cfg.block_kv, is_dkv=False)
  out = {}
  pmb = None if fwd.partial_mask_blocks is None else np.ascontiguousarray(fwd.partial_mask_blocks, dtype=np.int8)
  for name, kind in (("fwd", 0), ("dq", 1)):
    row_ptr, entries, row_order = splash._build_schedule(state, pid, cfg.block_q, cfg.block_kv, kind)  # pylint: disable=protected-access
    out[name] = dict(row_ptr=row_ptr, entries=entries, row_order=row_order, partial_mask_blocks=pmb)
  if dkv is not None:
    st2, pid2 = mask_info_lib.block_grids(dkv, q_len // cfg.block_q_dkv, kv_len // cfg.block_kv_dkv, is_dkv=True)
    pmb_t = None if dkv.partial_mask_blocks is None else np.ascontiguousarray(dkv.partial_mask_blocks, dtype=np.int8)
    row_ptr, entries, row_order = splash._build_schedule(st2, pid2, cfg.block_q_dkv, cfg.block_kv_dkv, 2)  # pylint: disable=protected-access
  else:
    pmb_t = None if pmb is None else np.ascontiguousarray(np.swapaxes(pmb, -1, -2))
    row_ptr, entries, row_order = splash._build_schedule(state, pid, cfg.block_q, cfg.block_kv, 2)  # pylint: disable=protected-access
  out["dkv"] = dict(row_ptr=row_ptr, entries=entries, row_order=row_order, partial_mask_blocks=pmb_t)
  return out


def _mask_attrs(kernel) -> dict[str, int]:
  rule = kernel.mask_function_rule
  names = ("kind", "offset", "left", "right", "has_left", "has_right", "chunk")
  if rule is None:
    return {f"mask_{n}": 0 for n in names}
  return {f"mask_{n}": int(getattr(rule, n)) for n in names}


def _empty(kind: str) -> np.ndarray:
  return np.zeros((0,), dtype=_NP_KIND[kind])


def call_plan(kernel, which: int, *, scale: float, layout: int = LAYOUT_BHSD, fused_backward: bool = True) -> dict:
  """Everything of a handler call that does not depend on the runtime tensors.

  Returns ``{"target", "operands": [(name, array-or-None)], "results": [names], "attrs": {...}}``:
  operands whose value is ``None`` are the runtime tensors the caller supplies (q, k, v, ...);
  optional operands that this kernel does not use are zero-element arrays, which the handler reads
  as NULL.  Attribute values are numpy scalars of the C type the handler declares.
  """
  sig = signature(which)
  scheds = host_schedules(kernel)
  cfg = kernel.config
  runtime = {"q", "k", "v", "o", "d_o", "logsumexp", "q_segment_ids", "kv_segment_ids", "sinks", "max_logit_value"}
  q_seq = np.asarray(kernel.fwd_mask_info.q_sequence) if kernel.fwd_mask_info.q_sequence is not None else None
  if q_seq is not None and np.array_equal(q_seq, np.arange(len(q_seq), dtype=q_seq.dtype)):
    q_seq = None
  operands = []
  for name, kind in sig["operands"]:
    if name in runtime:
      operands.append((name, None))
      continue
    if name == "q_sequence":
      value = q_seq
    else:
      which_sched, _, leaf = name.partition("_")
      value = scheds[{"sched": "fwd"}.get(which_sched, which_sched)].get(leaf) if leaf != "row_end" else None
    operands.append((name, _empty(kind) if value is None else np.ascontiguousarray(value, dtype=_NP_KIND[kind])))
  attrs = dict(_mask_attrs(kernel))
  attrs.update(layout=layout, scale=scale, soft_cap=float(cfg.attn_logits_soft_cap or 0.0),
               sched_block_q=cfg.block_q, sched_block_kv=cfg.block_kv)
  if which == FWD:
    attrs.update(mask_value=max(float(kernel.mask_value), -3.0e38), sched_entries_per_batch=0)
  else:
    attrs.update(flags=_native.BWD_FUSED_DQ if fused_backward else 0, dq_entries_per_batch=0, dkv_entries_per_batch=0)
  ctype = {"int32_t": np.int32, "int64_t": np.int64, "float": np.float32}
  typed = {name: ctype[t](attrs[name]) for name, t in sig["attrs"]}
  return {"target": TARGET_NAMES[which], "operands": operands, "results": [n for n, _ in sig["results"]], "attrs": typed}
