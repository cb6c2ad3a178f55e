"""Mask objects: lazy vs dense equality, algebra, hashing — the behaviours the reference's
splash_attention_mask_test.py:59-682 pins, on this package's classes."""
import numpy as np
import pytest

from tokamax_b200 import splash_attention_mask as m


def _full(mask):
  q, kv = mask.shape
  return np.asarray(mask[(slice(0, q), slice(0, kv))])


@pytest.mark.parametrize("shape", [(64, 64), (48, 96), (96, 48)])
@pytest.mark.parametrize("offset", [0, 5, -7])
def test_causal_lazy_equals_dense(shape, offset):
  np.testing.assert_array_equal(_full(m.CausalMask(shape, offset)), m.make_causal_mask(shape, offset))


@pytest.mark.parametrize("shape", [(64, 64), (48, 96), (96, 48)])
@pytest.mark.parametrize("window", [(8, 8), (8, None), (None, 3), (None, None), (0, 0)])
@pytest.mark.parametrize("offset", [0, 4, -3])
def test_local_lazy_equals_dense(shape, window, offset):
  np.testing.assert_array_equal(_full(m.LocalMask(shape, window, offset)),
                                m.make_local_attention_mask(shape, window, offset=offset))


@pytest.mark.parametrize("chunk", [1, 7, 16, 100])
def test_chunked_lazy_equals_dense(chunk):
  np.testing.assert_array_equal(_full(m.ChunkedCausalMask((64, 64), chunk)),
                                m.make_chunk_attention_mask((64, 64), chunk))
  with pytest.raises(ValueError):
    m.ChunkedCausalMask((8, 8), 0)
  with pytest.raises(ValueError):
    m.make_chunk_attention_mask((8, 8), -1)


def test_interval_rule_agrees_with_mask_function():
  for mask in (m.CausalMask((40, 56), 3), m.LocalMask((40, 56), (5, 2), -1), m.LocalMask((40, 56), (None, 2), 0),
               m.ChunkedCausalMask((40, 56), 12)):
    rule = mask.interval_rule
    dense = _full(mask)
    for i in range(40):
      lo, hi = -10**9, 10**9
      if rule.kind == m.KIND_CAUSAL:
        hi = i + rule.offset
      elif rule.kind == m.KIND_LOCAL:
        lo = i + rule.offset - rule.left if rule.has_left else lo
        hi = i + rule.offset + rule.right if rule.has_right else hi
      else:
        lo, hi = (i // rule.chunk) * rule.chunk, i
      want = np.array([lo <= j <= hi for j in range(56)])
      np.testing.assert_array_equal(dense[i], want)


def test_block_slices_and_unsupported_indices():
  mask = m.CausalMask((64, 64))
  np.testing.assert_array_equal(mask[(slice(16, 32), slice(8, 24))], m.make_causal_mask((64, 64))[16:32, 8:24])
  with pytest.raises(NotImplementedError):
    mask[(3, slice(0, 4))]
  with pytest.raises(NotImplementedError):
    m.FullMask((8, 8))[(slice(0, 4),)]


def test_algebra_shapes_bool_and_hash():
  a, b = m.CausalMask((32, 32)), m.LocalMask((32, 32), (4, 4), 0)
  np.testing.assert_array_equal(_full(a & b), _full(a) & _full(b))
  np.testing.assert_array_equal(_full(a | b), _full(a) | _full(b))
  with pytest.raises(ValueError):
    _ = a & m.CausalMask((16, 32))
  with pytest.raises(NotImplementedError):
    bool(a)
  with pytest.raises(NotImplementedError):
    _ = a and b
  assert a == m.CausalMask((32, 32)) and hash(a) == hash(m.CausalMask((32, 32)))
  assert a != m.CausalMask((32, 32), 1)
  assert (a & b) == (m.CausalMask((32, 32)) & m.LocalMask((32, 32), (4, 4), 0))
  assert hash(a & b) == hash(m.CausalMask((32, 32)) & m.LocalMask((32, 32), (4, 4), 0))
  assert hash(a & b) != hash(a | b)
  assert m.ChunkedCausalMask((32, 32), 8) == m.ChunkedCausalMask((32, 32), 8)
  assert m.ChunkedCausalMask((32, 32), 8) != m.ChunkedCausalMask((32, 32), 4)
  assert m.FullMask((4, 4)) == m.FullMask((4, 4)) and m.FullMask((4, 4)) != m.FullMask((4, 8))
  n1 = m.NumpyMask(np.eye(4, dtype=bool))
  assert n1 == m.NumpyMask(np.eye(4, dtype=bool)) and hash(n1) == hash(m.NumpyMask(np.eye(4, dtype=bool)))
  with pytest.raises(ValueError):
    m.NumpyMask(np.eye(4))
  with pytest.raises(ValueError):
    m.NumpyMask(np.ones((2, 2, 2), bool))
  with pytest.raises(ValueError):
    m.CausalMask((30, 30), shard_count=4)


def test_random_mask_is_reproducible():
  np.testing.assert_array_equal(m.make_random_mask((16, 16), 0.5, 3), m.make_random_mask((16, 16), 0.5, 3))
