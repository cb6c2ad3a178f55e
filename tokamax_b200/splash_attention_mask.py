"""Attention mask objects for splash attention.

Same public surface as the reference module
``tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_mask.py``:
``Mask`` (:27-55), the dense builders ``make_causal_mask`` (:58), ``make_local_attention_mask``
(:77), ``make_chunk_attention_mask`` (:96), ``make_random_mask`` (:125), the combinators
``LogicalOr`` / ``LogicalAnd`` (:133-174), the lazily evaluated ``CausalMask`` (:247),
``ChunkedCausalMask`` (:303), ``LocalMask`` (:363), and ``NumpyMask`` (:441), ``FullMask`` (:480).

The lazy masks are all expressed through one idea: query ``i`` keeps the keys of one closed
interval ``[lo(i), hi(i)]``.  That interval rule is what the CUDA kernels evaluate in registers
and what the native MaskInfo builder classifies blocks with, so each lazy mask also exports it
as a ``SplashMaskFn``-shaped tuple (``interval_rule``).
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, NamedTuple

import numpy as np


class IntervalRule(NamedTuple):
  """``[lo(i), hi(i)]`` description of a lazy mask (field order of the C struct SplashMaskFn)."""

  kind: int  # 1 causal, 2 local, 3 chunked
  offset: int = 0
  left: int = 0
  right: int = 0
  has_left: int = 0
  has_right: int = 0
  chunk: int = 0


KIND_CAUSAL, KIND_LOCAL, KIND_CHUNKED = 1, 2, 3


def _same_shape_or_raise(a: "Mask", b: "Mask") -> None:
  if a.shape != b.shape:
    raise ValueError(f"Invalid shape for other: {b.shape}, expected: {a.shape}")


class Mask:
  """Base class: a 2-D boolean mask that is only ever read through slices."""

  @property
  def shape(self) -> tuple[int, ...]:
    raise NotImplementedError

  def __getitem__(self, idx) -> np.ndarray:
    raise NotImplementedError

  def __bool__(self) -> bool:
    raise NotImplementedError(
        "Conversion to bool is unsupported. Could be caused by using logical"
        " instead of bitwise operations on masks."
    )

  def __or__(self, other: "Mask") -> "Mask":
    _same_shape_or_raise(self, other)
    return LogicalOr(self, other)

  def __and__(self, other: "Mask") -> "Mask":
    _same_shape_or_raise(self, other)
    return LogicalAnd(self, other)


# ----------------------------------------------------------------------------------------------
# dense builders
# ----------------------------------------------------------------------------------------------
def _index_grids(shape: tuple[int, int]) -> tuple[np.ndarray, np.ndarray]:
  q_len, kv_len = shape
  return (np.arange(q_len, dtype=np.int32)[:, None], np.arange(kv_len, dtype=np.int32)[None, :])


def make_causal_mask(shape: tuple[int, int], offset: int = 0) -> np.ndarray:
  """Dense causal mask: key ``j`` is kept for query ``i`` iff ``i + offset >= j``."""
  q, kv = _index_grids(shape)
  return (q + offset >= kv).astype(np.bool_)


def make_local_attention_mask(
    shape: tuple[int, int],
    window_size: tuple[int | None, int | None],
    *,
    offset: int = 0,
) -> np.ndarray:
  """Dense sliding-window mask; ``None`` leaves that side of the window open."""
  q, kv = _index_grids(shape)
  left, right = window_size
  keep = np.ones(shape, dtype=np.bool_)
  if left is not None:
    keep &= q - left + offset <= kv
  if right is not None:
    keep &= q + right + offset >= kv
  return keep


def make_chunk_attention_mask(shape: tuple[int, int], chunk_size: int) -> np.ndarray:
  """Dense chunked-causal mask: causal inside chunks of ``chunk_size``, nothing across."""
  if chunk_size <= 0:
    raise ValueError("chunk_size must be positive")
  q, kv = _index_grids(shape)
  return ((q // chunk_size) == (kv // chunk_size)) & (q >= kv)


def make_random_mask(shape: tuple[int, int], sparsity: float, seed: int) -> np.ndarray:
  """Bernoulli(1 - sparsity) mask from numpy's legacy global generator (as the reference)."""
  np.random.seed(seed)
  return np.random.binomial(n=1, p=1.0 - sparsity, size=shape).astype(np.bool_)


# ----------------------------------------------------------------------------------------------
# combinators
# ----------------------------------------------------------------------------------------------
class _Binary(Mask):
  """Elementwise combination of two masks of equal shape."""

  __slots__ = ("left", "right")
  _op: Callable[[np.ndarray, np.ndarray], np.ndarray]

  def __init__(self, left: Mask, right: Mask):
    if left.shape != right.shape:
      raise ValueError("Masks must have the same shape")
    self.left = left
    self.right = right

  @property
  def shape(self) -> tuple[int, ...]:
    return self.left.shape

  def __getitem__(self, idx) -> np.ndarray:
    return type(self)._op(self.left[idx], self.right[idx])

  def __eq__(self, other: object):
    if type(other) is not type(self):
      return NotImplemented
    return self.left == other.left and self.right == other.right

  def __hash__(self):
    return hash((type(self), self.left, self.right))

  def __repr__(self):
    return f"{type(self).__name__}(left={self.left!r}, right={self.right!r})"


class LogicalOr(_Binary):
  _op = staticmethod(np.logical_or)


class LogicalAnd(_Binary):
  _op = staticmethod(np.logical_and)


# ----------------------------------------------------------------------------------------------
# lazily evaluated masks
# ----------------------------------------------------------------------------------------------
def _resolve_slice(s: slice, size: int) -> slice:
  if s.step not in (None, 1):
    raise AssertionError("strided mask slices are not supported")
  start = 0 if s.start is None else s.start
  stop = size if s.stop is None else s.stop
  assert 0 <= start and stop <= size
  return slice(start, stop)


def _two_slices(idx, shape) -> tuple[slice, slice]:
  if len(idx) != 2 or not all(isinstance(s, slice) for s in idx):
    raise NotImplementedError(f"Unsupported slice: {idx}")
  return _resolve_slice(idx[0], shape[0]), _resolve_slice(idx[1], shape[1])


class _ComputableMask(Mask):
  """A mask given by a function of (q index, kv index), evaluated on demand.

  Attributes:
    q_sequence: ``int32[q_seq_len]`` token index of every q row (``arange``).
    mask_function: callable ``(q_ids[:, None], kv_ids[None, :]) -> bool array``; the kernels
      evaluate the equivalent ``interval_rule`` instead of loading mask data.
  """

  _shape: tuple[int, int]
  q_sequence: np.ndarray
  mask_function: Callable[..., Any]

  def __init__(self, shape: tuple[int, int], mask_function: Callable[..., Any], shard_count: int = 1):
    self._shape = shape
    self.mask_function = mask_function
    if shape[0] % (shard_count * shard_count) != 0:
      raise ValueError(
          f"Shard count squared ({shard_count * shard_count}) must"
          f" divide Q seq_len ({shape[0]}) evenly."
      )
    self.q_sequence = np.arange(shape[0], dtype=np.int32)

  @property
  def shape(self) -> tuple[int, ...]:
    return self._shape

  @property
  def interval_rule(self) -> IntervalRule:
    raise NotImplementedError

  def __getitem__(self, idx) -> np.ndarray:
    q_slice, kv_slice = _two_slices(idx, self.shape)
    rows = self.q_sequence[q_slice]
    cols = np.arange(kv_slice.start, kv_slice.stop)
    return self.mask_function(rows[:, None], cols[None, :])

  def _identity(self) -> tuple:
    raise NotImplementedError

  def __eq__(self, other: object):
    if type(self) is _ComputableMask:
      raise NotImplementedError()
    if not isinstance(other, type(self)):
      return NotImplemented
    return self._identity() == other._identity() and np.array_equal(self.q_sequence, other.q_sequence)

  def __hash__(self):
    if type(self) is _ComputableMask:
      raise NotImplementedError()
    return hash((type(self),) + self._identity() + (self.q_sequence.tobytes(),))


class CausalMask(_ComputableMask):
  """Lazy causal mask: query ``i`` sees keys ``j <= i + offset``."""

  offset: int

  def __init__(self, shape: tuple[int, int], offset: int = 0, shard_count: int = 1):
    self.offset = offset

    def causal_mask_function(q_ids, kv_ids):
      return q_ids >= kv_ids if self.offset == 0 else q_ids + self.offset >= kv_ids

    super().__init__(shape=shape, mask_function=causal_mask_function, shard_count=shard_count)

  @property
  def interval_rule(self) -> IntervalRule:
    return IntervalRule(KIND_CAUSAL, offset=int(self.offset))

  def _identity(self):
    return (self.shape, self.offset)


class ChunkedCausalMask(_ComputableMask):
  """Lazy chunked causal mask: causal inside ``chunk_size`` blocks, nothing across blocks."""

  chunk_size: int

  def __init__(self, shape: tuple[int, int], chunk_size: int, shard_count: int = 1):
    if chunk_size <= 0:
      raise ValueError("chunk_size must be positive")
    self.chunk_size = chunk_size

    def chunked_causal_mask_function(q_ids, kv_ids):
      return ((q_ids // self.chunk_size) == (kv_ids // self.chunk_size)) & (q_ids >= kv_ids)

    super().__init__(shape=shape, mask_function=chunked_causal_mask_function, shard_count=shard_count)

  @property
  def interval_rule(self) -> IntervalRule:
    return IntervalRule(KIND_CHUNKED, chunk=int(self.chunk_size))

  def _identity(self):
    return (self.shape, self.chunk_size)


class LocalMask(_ComputableMask):
  """Lazy sliding-window mask: ``i + offset - left <= j <= i + offset + right``."""

  window_size: tuple[int | None, int | None]
  offset: int

  def __init__(
      self,
      shape: tuple[int, int],
      window_size: tuple[int | None, int | None],
      offset: int,
      shard_count: int = 1,
  ):
    self.window_size = window_size
    self.offset = offset

    def local_mask_function(q_ids, kv_ids):
      left, right = self.window_size
      assert q_ids.ndim == 2 and kv_ids.ndim == 2
      if left is None and right is None:
        return np.ones((q_ids.shape[0], kv_ids.shape[1]), dtype=np.bool_)
      shifted = q_ids + self.offset if self.offset != 0 else q_ids
      keep = None
      if left is not None:
        keep = shifted - left <= kv_ids
      if right is not None:
        upper = shifted + right >= kv_ids
        keep = upper if keep is None else keep & upper
      return keep

    super().__init__(shape=shape, mask_function=local_mask_function, shard_count=shard_count)

  @property
  def interval_rule(self) -> IntervalRule:
    left, right = self.window_size
    return IntervalRule(
        KIND_LOCAL,
        offset=int(self.offset),
        left=int(left or 0),
        right=int(right or 0),
        has_left=int(left is not None),
        has_right=int(right is not None),
    )

  def _identity(self):
    return (self.shape, self.window_size, self.offset)

  def __eq__(self, other: object):
    if not isinstance(other, type(self)):
      return False
    return super().__eq__(other)

  __hash__ = _ComputableMask.__hash__


# ----------------------------------------------------------------------------------------------
# dense and full masks
# ----------------------------------------------------------------------------------------------
@dataclasses.dataclass(slots=True)
class NumpyMask(Mask):
  """A mask backed by a dense boolean numpy array."""

  array: np.ndarray

  def __post_init__(self):
    if self.array.ndim != 2:
      raise ValueError("Expected a 2-dim array")
    if self.array.dtype != np.bool_:
      raise ValueError("Mask must be a boolean array")

  @property
  def shape(self) -> tuple[int, ...]:
    return self.array.shape

  def __getitem__(self, idx) -> np.ndarray:
    return self.array[idx]

  def __eq__(self, other: object):
    if not isinstance(other, type(self)):
      return NotImplemented
    return np.array_equal(self.array, other.array, equal_nan=True)

  def __hash__(self):
    return hash((type(self), self.array.tobytes()))


@dataclasses.dataclass(frozen=True, slots=True)
class FullMask(Mask):
  """Lazy all-ones mask."""

  _shape: tuple[int, int]

  def __post_init__(self):
    if not isinstance(self.shape, tuple):
      raise ValueError(f"Unsupported shape type: {type(self.shape)}")

  @property
  def shape(self) -> tuple[int, ...]:
    return self._shape

  def __getitem__(self, idx) -> np.ndarray:
    i, j = _two_slices(idx, self.shape)
    return np.ones((i.stop - i.start, j.stop - j.start), dtype=np.bool_)

  def __eq__(self, other: object):
    if not isinstance(other, type(self)):
      return NotImplemented
    return self.shape == other.shape

  def __hash__(self):
    return hash((type(self), self.shape))
