"""Case list shared by the golden-vector generator and the MaskInfo tests.

A mask spec is a nested list: ["causal", q, kv, offset], ["local", q, kv, left, right, offset]
(left / right may be None), ["chunked", q, kv, chunk], ["full", q, kv], ["dense", <spec>]
(the same mask materialised into a NumpyMask), ["random", q, kv, sparsity, seed],
["and", a, b], ["or", a, b], ["vstack", a, b] / ["hstack", a, b] (dense concatenation).
"""

from __future__ import annotations

import numpy as np


def build_mask(spec, lib):
  """Instantiates ``spec`` with the mask classes of module ``lib``."""
  kind = spec[0]
  if kind == "causal":
    return lib.CausalMask((spec[1], spec[2]), spec[3])
  if kind == "local":
    return lib.LocalMask((spec[1], spec[2]), (spec[3], spec[4]), spec[5])
  if kind == "chunked":
    return lib.ChunkedCausalMask((spec[1], spec[2]), spec[3])
  if kind == "full":
    return lib.FullMask((spec[1], spec[2]))
  if kind == "random":
    return lib.NumpyMask(lib.make_random_mask((spec[1], spec[2]), spec[3], spec[4]))
  if kind == "dense":
    inner = build_mask(spec[1], lib)
    q, kv = inner.shape
    return lib.NumpyMask(np.asarray(inner[(slice(0, q), slice(0, kv))]).astype(np.bool_))
  if kind in ("and", "or"):
    a, b = build_mask(spec[1], lib), build_mask(spec[2], lib)
    return a & b if kind == "and" else a | b
  if kind in ("vstack", "hstack"):
    a, b = (build_mask(["dense", s], lib).array for s in spec[1:3])
    return lib.NumpyMask(np.concatenate([a, b], axis=0 if kind == "vstack" else 1))
  raise ValueError(f"unknown mask spec {spec!r}")


def _case(name, mask, block, *, q_shards=1, kv_shards=1, dkv_dynamic=False, downcast=True, digest=False):
  return dict(name=name, mask=mask, block=list(block), q_shards=q_shards, kv_shards=kv_shards,
              dkv_dynamic=dkv_dynamic, downcast=downcast, digest=digest)


# Small cases follow the shapes the reference's own MaskInfo tests use
# (splash_attention_mask_test.py:752-1660: 16x16 blocks, wide / tall rectangles, local windows,
# stacked shards, 2x2 shards); stored in full.
CASES = [
    _case("full_lazy", ["full", 64, 64], (16, 16)),
    _case("full_dense", ["dense", ["full", 64, 64]], (16, 16)),
    _case("no_partial_blocks", ["dense", ["chunked", 64, 64, 16]], (16, 16)),
    _case("causal_square_lazy", ["causal", 64, 64, 0], (16, 16)),
    _case("causal_square_dense", ["dense", ["causal", 64, 64, 0]], (16, 16)),
    _case("causal_wide_lazy", ["causal", 64, 128, 0], (16, 16)),
    _case("causal_wide_dense_dyn", ["dense", ["causal", 64, 128, 0]], (16, 16), dkv_dynamic=True),
    _case("causal_tall_lazy", ["causal", 128, 64, 0], (16, 16)),
    _case("causal_tall_dense", ["dense", ["causal", 128, 64, 0]], (16, 16), dkv_dynamic=True),
    _case("causal_offset_pos", ["causal", 64, 64, 7], (16, 16)),
    _case("causal_offset_neg_dense", ["dense", ["causal", 64, 96, -5]], (16, 32), dkv_dynamic=True),
    _case("local_lazy", ["local", 64, 64, 8, 8, 0], (16, 16)),
    _case("local_dense", ["dense", ["local", 64, 64, 8, 8, 0]], (16, 16)),
    _case("local_narrow_lazy", ["local", 64, 64, 8, 0, 0], (16, 16)),
    _case("local_narrow_dense", ["dense", ["local", 64, 64, 8, 0, 0]], (16, 16), dkv_dynamic=True),
    _case("local_left_only", ["local", 96, 96, 20, None, 0], (16, 16)),
    _case("local_right_only_dense", ["dense", ["local", 96, 96, None, 12, 3]], (16, 16)),
    _case("chunked_lazy", ["chunked", 128, 128, 32], (16, 16)),
    _case("chunked_odd_dense", ["dense", ["chunked", 96, 96, 24]], (16, 16), dkv_dynamic=True),
    _case("and_local_causal", ["and", ["local", 128, 128, 40, None, 0], ["causal", 128, 128, 0]], (16, 16)),
    _case("or_local_chunked", ["or", ["local", 128, 128, 4, 4, 0], ["chunked", 128, 128, 32]], (32, 16),
          dkv_dynamic=True),
    _case("and_random_causal", ["and", ["random", 128, 128, 0.5, 3], ["causal", 128, 128, 0]], (32, 32)),
    _case("random_sparse", ["random", 128, 256, 0.97, 1], (16, 32), dkv_dynamic=True),
    _case("random_dense_rows_empty", ["random", 64, 64, 0.995, 11], (16, 16), dkv_dynamic=True),
    _case("qshards2_causal_local", ["vstack", ["causal", 64, 64, 0], ["local", 64, 64, 8, 8, 0]], (16, 16),
          q_shards=2),
    _case("qshards2_wide_narrow", ["vstack", ["local", 64, 64, 8, 8, 0], ["local", 64, 64, 8, 0, 0]], (16, 16),
          q_shards=2, dkv_dynamic=True),
    _case("kvshards2_wide_narrow", ["hstack", ["local", 64, 64, 8, 8, 0], ["local", 64, 64, 8, 0, 0]], (16, 16),
          kv_shards=2),
    _case("causal_2x2_shards_dyn", ["dense", ["causal", 128, 128, 0]], (16, 16), q_shards=2, kv_shards=2,
          dkv_dynamic=True),
    _case("causal_2x2_shards_static", ["dense", ["causal", 128, 128, 0]], (16, 16), q_shards=2, kv_shards=2),
    _case("causal_lazy_4qshards", ["causal", 256, 256, 0], (16, 32), q_shards=4, dkv_dynamic=True),
    _case("no_downcast", ["dense", ["causal", 64, 64, 0]], (16, 16), downcast=False, dkv_dynamic=True),
    # full blocks after the last partial one: the reference's walk over the partial blocks runs out
    # and stays on the first of them (mask_info.py:208-223)
    _case("full_blocks_after_last_partial", ["or", ["chunked", 512, 512, 512], ["local", 512, 512, 128, 200, 9]],
          (128, 256)),
    _case("full_blocks_after_last_partial_dyn", ["or", ["chunked", 512, 512, 512], ["local", 512, 512, 128, 200, 9]],
          (128, 128), dkv_dynamic=True),
    _case("full_blocks_after_last_partial_kvshards", ["or", ["causal", 512, 512, 0], ["random", 512, 512, 0.5, 7]],
          (128, 128), kv_shards=2, downcast=False),
    # int16 indices: more than 128 blocks per side
    _case("causal_int16_index", ["causal", 4096, 4096, 0], (16, 16), dkv_dynamic=True, digest=True),
    # the benchmark configurations at the kernels' 128x128 blocks; stored as digests
    _case("c1_causal_1024", ["causal", 1024, 1024, 0], (128, 128)),
    _case("c2_causal_8192", ["causal", 8192, 8192, 0], (128, 128), digest=True),
    _case("c2_causal_8192_dyn", ["causal", 8192, 8192, 0], (128, 128), dkv_dynamic=True, digest=True),
    _case("c3_local_4096_16384", ["local", 16384, 16384, 4096, 0, 0], (128, 128), digest=True),
    _case("c3_composed_2048", ["and", ["local", 2048, 2048, 512, None, 0], ["causal", 2048, 2048, 0]],
          (128, 128), dkv_dynamic=True),
    _case("c5_causal_32768", ["causal", 32768, 32768, 0], (128, 128), digest=True),
    _case("c4_causal_131072_b1024", ["causal", 131072, 131072, 0], (1024, 1024), digest=True),
    _case("c4_causal_131072", ["causal", 131072, 131072, 0], (128, 128), digest=True),
]

FIELDS = ("mask_next", "active_rows", "active_cols", "block_mask", "num_active_blocks",
          "partial_mask_blocks", "q_sequence")
