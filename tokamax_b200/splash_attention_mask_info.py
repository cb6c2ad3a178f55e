"""MaskInfo: block-sparse description of an attention mask.

Public surface of the reference module
``tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_mask_info.py``:
``MaskInfo`` (:51-88), ``process_mask`` / ``process_mask_dkv`` (:573-574, ``_process_mask``
:357-570), ``find_bounds`` (:33-47) and the small-dtype rule ``_downcast_to_small_type`` (:91-124).

The tables are produced by the native builder ``splash_maskinfo_build`` (C++, analytic block
classification); this module only flattens the mask expression into the node list the C ABI
takes, applies the dtype rule and caches results the way the reference does (``lru_cache``).
Tables are bit-identical to the reference's, including dtypes and which fields are ``None``.
"""

from __future__ import annotations

import ctypes as C
import functools
from typing import Any, Callable, NamedTuple

import numpy as np

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_mask as mask_lib

MaskCallable = Any


class MaskInfo(NamedTuple):
  """Block-sparse tables consumed by the splash kernels.

  Attributes:
    mask_next: integer[n] id into ``partial_mask_blocks`` of the partial block at or after
      each step, or None.
    active_rows / active_cols: integer[n] block coordinates of each step (dynamic grid), or
      None (static grid / all-full mask).  For the dkv table rows are kv blocks.
    block_mask: integer[n]; 0 empty, 1 partially masked, 2 full (-1 = shard padding).
    num_active_blocks: int32[n_shards] number of valid steps per shard, or None.
    partial_mask_blocks: int8[n_partial, block_q, block_kv] unique partially-masked blocks
      ([n_partial, block_kv, block_q] for dkv), or None.
    q_sequence: int32[q_seq_len] for masks evaluated in-kernel, else None.
  """

  mask_next: np.ndarray | None
  active_rows: np.ndarray | None
  active_cols: np.ndarray | None
  block_mask: np.ndarray | None
  num_active_blocks: np.ndarray | None
  partial_mask_blocks: np.ndarray | None
  q_sequence: np.ndarray | None


def find_bounds(arr):
  """Row-start / row-end flags of a step list: 1 where the value differs from its neighbour.

  The first entry of ``bounds_start`` and the last of ``bounds_end`` are forced to 1.
  Accepts numpy arrays or torch tensors; ``None`` gives ``(None, None)``.
  """
  if arr is None:
    return None, None
  try:
    import torch  # pylint: disable=g-import-not-at-top

    if isinstance(arr, torch.Tensor):
      start = (arr != torch.roll(arr, 1, -1)).to(torch.int32)
      end = (arr != torch.roll(arr, -1, -1)).to(torch.int32)
      start[..., 0] = 1
      end[..., -1] = 1
      return start, end
  except ImportError:  # pragma: no cover
    pass
  arr = np.asarray(arr)
  start = (arr != np.roll(arr, 1, axis=-1)).astype(np.int32)
  end = (arr != np.roll(arr, -1, axis=-1)).astype(np.int32)
  start[..., 0] = 1
  end[..., -1] = 1
  return start, end


def _downcast_to_small_type(array: np.ndarray) -> np.ndarray:
  """int32 -> int8 / int16 when every value fits (values below -1 are rejected)."""
  if array.dtype != np.int32:
    raise ValueError(f"Expected int32 input, but got {array.dtype}.")
  if not np.all(array >= -1):
    raise ValueError("Expected non-negative array.")
  if array.size == 0:
    return array
  top = int(array.max())
  if top <= np.iinfo(np.int8).max:
    return array.astype(np.int8)
  if top <= np.iinfo(np.int16).max:
    return array.astype(np.int16)
  return array


def _check_mask(mask: mask_lib.Mask) -> None:
  """Rejects masks with an all-zero row (the softmax of that row would divide by zero)."""
  assert len(mask.shape) == 2
  q_len, kv_len = mask.shape
  row_live = np.zeros(q_len, dtype=np.bool_)
  band = 4096
  for c0 in range(0, kv_len, band):
    row_live |= np.asarray(mask[(slice(0, q_len), slice(c0, min(kv_len, c0 + band)))]).any(axis=1)
  if not row_live.all():
    raise ValueError(
        "Some rows of the mask (along the kv dimension) are all zeros.\nThis is"
        " would result in a division by zero when computing the attention"
        " softmax."
    )


def _process_dynamic_mask(
    mask,
    block_shape: tuple[int, int],
    is_dkv: bool,
    *,
    downcast_smem_data: bool = True,
    partial_mask_blocks_dtype: Any = np.int8,
) -> MaskInfo:
  """MaskInfo of a mask only known at run time (one shard, fixed-size tables).

  Counterpart of the reference's ``_process_dynamic_mask`` (mask_info.py:231-350): every block
  keeps a slot (no deduplication), steps are the active blocks in row-major order padded with
  -1 to ``n_q_blocks * n_kv_blocks`` entries, ``mask_next`` is the block's own linear id where
  it is partial and 0 elsewhere.  ``mask`` is a bool array (numpy, or a torch tensor on any
  device).
  """
  if hasattr(mask, "detach"):
    mask = mask.detach().cpu().numpy()
  mask = np.asarray(mask)
  if mask.ndim != 2:
    raise ValueError(f"Expected a 2-dim mask, instead got: {mask.shape}.")
  q_seq_len, kv_seq_len = mask.shape
  q_block_size, kv_block_size = block_shape
  if q_seq_len % q_block_size != 0:
    raise ValueError(f"{q_block_size=} should divide {q_seq_len=}.")
  if kv_seq_len % kv_block_size != 0:
    raise ValueError(f"{kv_block_size=} should divide {kv_seq_len=}.")
  nq, nkv = q_seq_len // q_block_size, kv_seq_len // kv_block_size
  blocks = mask.reshape(nq, q_block_size, nkv, kv_block_size).swapaxes(1, 2).astype(partial_mask_blocks_dtype)
  state = blocks.any(axis=(-1, -2)).astype(np.int32) + blocks.all(axis=(-1, -2)).astype(np.int32)
  ids = np.arange(nq * nkv, dtype=np.int32).reshape(nq, nkv)
  if is_dkv:
    state, ids, blocks = state.T, ids.T, blocks.swapaxes(-1, -2)
  active = state > 0
  if is_dkv:
    active = active | ((~active.any(axis=1))[:, None] & (np.arange(state.shape[1]) == 0)[None, :])
  n_active = int(active.sum())
  total = nq * nkv
  coords = np.argwhere(active)
  active_rows = np.full(total, -1, np.int32)
  active_cols = np.full(total, -1, np.int32)
  active_rows[:n_active] = coords[:, 0]
  active_cols[:n_active] = coords[:, 1]
  # Padding slots read element [-1, -1], as negative indices do in the reference.
  block_mask = state[active_rows, active_cols].astype(np.int32)
  # The reference gathers the ids without wrapping negative indices, which yields the most
  # negative int32 on padding slots; the int8 / int16 downcast below then truncates that to 0.
  gathered = np.where(active_rows >= 0, ids[active_rows, active_cols], np.iinfo(np.int32).min)
  mask_next = np.where(block_mask == 1, gathered, 0).astype(np.int32)
  block_mask = block_mask * (np.arange(total) < n_active).astype(np.int32)
  partial_mask_blocks = blocks.reshape((total,) + blocks.shape[2:])
  if downcast_smem_data:
    block_mask = block_mask.astype(np.int8)
    if total <= 127:
      mask_next = mask_next.astype(np.int8)
    elif total <= 32767:
      mask_next = mask_next.astype(np.int16)
  return MaskInfo(
      mask_next=mask_next,
      active_rows=active_rows,
      active_cols=active_cols,
      block_mask=block_mask,
      num_active_blocks=np.array([n_active], dtype=np.int32),
      partial_mask_blocks=partial_mask_blocks,
      q_sequence=None,
  )


# ----------------------------------------------------------------------------------------------
# mask expression -> node list
# ----------------------------------------------------------------------------------------------
_NODE_FULL, _NODE_CAUSAL, _NODE_LOCAL, _NODE_CHUNKED, _NODE_DENSE, _NODE_AND, _NODE_OR = range(7)
_KIND_TO_NODE = {
    mask_lib.KIND_CAUSAL: _NODE_CAUSAL,
    mask_lib.KIND_LOCAL: _NODE_LOCAL,
    mask_lib.KIND_CHUNKED: _NODE_CHUNKED,
}


def _fill_fn(dst: _native.SplashMaskFn, rule: mask_lib.IntervalRule) -> None:
  for name, value in zip(rule._fields, rule):
    setattr(dst, name, int(value))


def _dense_from(mask: mask_lib.Mask) -> np.ndarray:
  """Materialises an arbitrary Mask through its slicing interface (row bands of 1024)."""
  q_len, kv_len = mask.shape
  out = np.empty((q_len, kv_len), dtype=np.bool_)
  band = 1024
  for r0 in range(0, q_len, band):
    r1 = min(q_len, r0 + band)
    out[r0:r1] = mask[(slice(r0, r1), slice(0, kv_len))]
  return out


def _flatten(mask: mask_lib.Mask, nodes: list, keepalive: list) -> int:
  """Appends ``mask`` (children first) to ``nodes``; returns its index."""
  node = _native.SplashMaskNode()
  node.left_child = node.right_child = -1
  if isinstance(mask, (mask_lib.LogicalAnd, mask_lib.LogicalOr)):
    left = _flatten(mask.left, nodes, keepalive)
    right = _flatten(mask.right, nodes, keepalive)
    node.kind = _NODE_AND if isinstance(mask, mask_lib.LogicalAnd) else _NODE_OR
    node.left_child, node.right_child = left, right
  elif isinstance(mask, mask_lib.FullMask):
    node.kind = _NODE_FULL
  elif isinstance(mask, mask_lib._ComputableMask) and np.array_equal(  # pylint: disable=protected-access
      mask.q_sequence, np.arange(mask.shape[0], dtype=np.int32)
  ):
    rule = mask.interval_rule
    node.kind = _KIND_TO_NODE[rule.kind]
    _fill_fn(node.fn, rule)
  else:
    dense = mask.array if isinstance(mask, mask_lib.NumpyMask) else _dense_from(mask)
    dense = np.ascontiguousarray(dense, dtype=np.bool_)
    keepalive.append(dense)
    node.kind = _NODE_DENSE
    node.dense = dense.ctypes.data
  nodes.append(node)
  return len(nodes) - 1


def _copy_out(ptr, count: int) -> np.ndarray | None:
  if not ptr:
    return None
  if count == 0:
    return np.zeros((0,), dtype=np.int32)
  return np.ctypeslib.as_array(ptr, shape=(count,)).copy()


@functools.lru_cache(maxsize=12)
def _process_mask(
    mask: mask_lib.Mask,
    block_shape: tuple[int, int],
    is_dkv: bool,
    *,
    downcast_smem_data: bool = True,
    partial_mask_blocks_dtype: Any = np.int8,
    q_seq_shards: int = 1,
    kv_seq_shards: int = 1,
    return_dynamic_grid: bool = True,
) -> tuple[MaskInfo, MaskCallable | None]:
  """Turns a mask into ``(MaskInfo, mask_function or None)``.

  Raises ValueError for a non-2D mask or block / shard counts that do not divide the sequence
  lengths (same conditions and order as the reference).
  """
  if len(mask.shape) != 2:
    raise ValueError(f"Expected a 2-dim mask, instead got: {mask.shape=}")
  q_seq_len, kv_seq_len = mask.shape
  q_block_size, kv_block_size = block_shape
  if q_seq_len % q_block_size != 0:
    raise ValueError(f"{q_block_size=} should divide {q_seq_len=}.")
  if kv_seq_len % kv_block_size != 0:
    raise ValueError(f"{kv_block_size=} should divide {kv_seq_len=}.")
  q_seq_len_per_shard, rem = divmod(q_seq_len, q_seq_shards)
  if rem != 0:
    raise ValueError(f"{q_seq_shards=} should divide {q_seq_len=}.")
  if q_seq_len_per_shard % q_block_size != 0:
    raise ValueError(f"{q_block_size=} should divide {q_seq_len_per_shard=}.")
  kv_seq_len_per_shard, rem = divmod(kv_seq_len, kv_seq_shards)
  if rem != 0:
    raise ValueError(f"{kv_seq_shards=} should divide {kv_seq_len=}.")
  if kv_seq_len_per_shard % kv_block_size != 0:
    raise ValueError(f"{kv_block_size=} should divide {kv_seq_len_per_shard=}.")

  assert hasattr(mask, "q_sequence") == hasattr(mask, "mask_function")
  if hasattr(mask, "q_sequence"):
    q_sequence, mask_function = mask.q_sequence, mask.mask_function
  else:
    q_sequence = mask_function = None

  nodes: list = []
  keepalive: list = []
  _flatten(mask, nodes, keepalive)
  node_array = (_native.SplashMaskNode * len(nodes))(*nodes)
  out = _native.SplashMaskInfoOut()
  lib = _native.lib()
  _native.check(
      lib.splash_maskinfo_build(
          node_array, len(nodes), q_seq_len, kv_seq_len, q_block_size, kv_block_size, int(is_dkv),
          q_seq_shards, kv_seq_shards, int(return_dynamic_grid), C.byref(out)),
      "splash_maskinfo_build",
  )
  try:
    if out.all_full:
      return MaskInfo(None, None, None, None, None, None, q_sequence), None
    n = int(out.n_entries)
    mask_next = _copy_out(out.mask_next, n)
    active_rows = _copy_out(out.active_rows, n)
    active_cols = _copy_out(out.active_cols, n)
    block_mask = _copy_out(out.block_mask, n)
    num_active_blocks = _copy_out(out.num_active_blocks, int(out.n_shards))
    partial_mask_blocks = None
    if out.partial_mask_blocks:
      pm_shape = (kv_block_size, q_block_size) if is_dkv else (q_block_size, kv_block_size)
      partial_mask_blocks = (
          np.ctypeslib.as_array(out.partial_mask_blocks, shape=(int(out.n_partial),) + pm_shape)
          .copy()
          .astype(partial_mask_blocks_dtype)
      )
  finally:
    lib.splash_maskinfo_free(C.byref(out))

  if downcast_smem_data:
    if active_rows is not None:
      active_rows = _downcast_to_small_type(active_rows)
      active_cols = _downcast_to_small_type(active_cols)
    if mask_next is not None:
      mask_next = _downcast_to_small_type(mask_next)
    block_mask = _downcast_to_small_type(block_mask)

  assert (mask_function is not None) == (q_sequence is not None)
  return (
      MaskInfo(
          mask_next=mask_next if mask_function is None else None,
          active_rows=active_rows,
          active_cols=active_cols,
          block_mask=block_mask,
          num_active_blocks=num_active_blocks,
          partial_mask_blocks=partial_mask_blocks if mask_function is None else None,
          q_sequence=q_sequence,
      ),
      mask_function,
  )


process_mask = functools.partial(_process_mask, is_dkv=False)
process_mask_dkv = functools.partial(_process_mask, is_dkv=True)

process_dynamic_mask = functools.partial(_process_dynamic_mask, is_dkv=False)
process_dynamic_mask_dkv = functools.partial(_process_dynamic_mask, is_dkv=True)


# ----------------------------------------------------------------------------------------------
# MaskInfo -> block grids (what the kernel schedule is cut from)
# ----------------------------------------------------------------------------------------------
def block_grids(
    info: MaskInfo, n_q_blocks: int, n_kv_blocks: int, *, is_dkv: bool, shard: int = 0, n_shards: int = 1
) -> tuple[np.ndarray, np.ndarray]:
  """Rebuilds ``(state[n_q_blocks, n_kv_blocks], partial_id[...])`` from a MaskInfo.

  ``state`` is 0 / 1 / 2 per block in (q block, kv block) orientation whatever table it came
  from; ``partial_id`` is the ``partial_mask_blocks`` index of partial blocks, else -1.  For tables
  built with ``q_seq_shards = n_shards > 1`` (reference :494-544: one padded segment per shard,
  shard-local indices) ``shard`` selects the segment and ``n_q_blocks`` counts that shard's q blocks.
  """
  if not 0 <= shard < n_shards:
    raise ValueError(f"shard {shard} out of range for {n_shards} shards")
  if info.block_mask is None:  # all-full mask
    return (np.full((n_q_blocks, n_kv_blocks), 2, np.int32), np.full((n_q_blocks, n_kv_blocks), -1, np.int32))
  shape = (n_kv_blocks, n_q_blocks) if is_dkv else (n_q_blocks, n_kv_blocks)
  block_mask = np.asarray(info.block_mask).astype(np.int32)
  mask_next = None if info.mask_next is None else np.asarray(info.mask_next).astype(np.int32)
  if block_mask.size % n_shards != 0:
    raise ValueError(f"a table of {block_mask.size} entries does not split into {n_shards} shards")
  seg = block_mask.size // n_shards
  lo = shard * seg
  block_mask = block_mask[lo:lo + seg]
  if mask_next is not None:
    mask_next = mask_next[lo:lo + seg]
  state = np.zeros(shape, np.int32)
  pid = np.full(shape, -1, np.int32)
  if info.active_rows is not None:
    counts = info.num_active_blocks
    if counts is not None and len(counts) != n_shards:
      raise ValueError(f"the MaskInfo holds {len(counts)} shards, the caller expects {n_shards}")
    n = int(counts[shard]) if counts is not None else block_mask.size
    rows = np.asarray(info.active_rows).astype(np.int64)[lo:lo + n]
    cols = np.asarray(info.active_cols).astype(np.int64)[lo:lo + n]
    state[rows, cols] = block_mask[:n]
    if mask_next is not None:
      part = block_mask[:n] == 1
      pid[rows[part], cols[part]] = mask_next[:n][part]
  else:
    if block_mask.size != shape[0] * shape[1]:
      raise ValueError(f"a static grid of {block_mask.size} blocks per shard does not match {shape}")
    state = block_mask.reshape(shape).copy()
    if mask_next is not None:
      pid = np.where(state == 1, mask_next.reshape(shape), -1).astype(np.int32)
  if is_dkv:
    state, pid = state.T, pid.T
  return np.ascontiguousarray(state), np.ascontiguousarray(pid)
