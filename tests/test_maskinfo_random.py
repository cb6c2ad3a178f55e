"""Seeded random masks: the native MaskInfo builder against the CPU restatement of the reference's
builder (two independent implementations: analytic C++ and a block-by-block numpy loop), and —
where a checkout of the reference is at hand (SPLASH_REFERENCE_ROOT) — both against the reference's
own code.  Values, dtypes, shapes and None-ness must agree exactly.

The draw covers what the golden cases fix only in a few points: composed masks two levels deep,
unequal q / kv lengths, block shapes from 16 to 512, q / kv shards, static and dynamic grids, and in
particular masks whose last blocks are full (the walk over the partial blocks that fills
`mask_next` then runs out, reference mask_info.py:208-223).
"""
import random

import numpy as np
import pytest

from oracle import maskinfo_ref
from oracle import ref_loader
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import splash_attention_mask_info as mask_info_lib

FIELDS = mask_info_lib.MaskInfo._fields


def _leaf(rng, sq, skv):
  kind = rng.choice(["causal", "local", "chunked", "full", "dense"])
  if kind == "causal":
    return ("causal", rng.choice([0, 0, skv - sq, 17, -33]))
  if kind == "local":
    return ("local", rng.choice([None, 40, 128, 300]), rng.choice([None, 0, 64, 200]), rng.choice([0, 9, -20]))
  if kind == "chunked":
    return ("chunked", rng.choice([32, 128, 200, 512]))
  if kind == "full":
    return ("full",)
  return ("dense", rng.randint(0, 10**6), rng.choice([0.1, 0.5, 0.9]))


def _make(spec, lib, sq, skv):
  if spec[0] == "causal":
    return lib.CausalMask((sq, skv), offset=spec[1])
  if spec[0] == "local":
    return lib.LocalMask((sq, skv), (spec[1], spec[2]), spec[3])
  if spec[0] == "chunked":
    return lib.ChunkedCausalMask((sq, skv), spec[1])
  if spec[0] == "full":
    return lib.FullMask((sq, skv))
  if spec[0] == "dense":
    return lib.NumpyMask(np.random.default_rng(spec[1]).random((sq, skv)) < spec[2])
  a, b = _make(spec[1], lib, sq, skv), _make(spec[2], lib, sq, skv)
  return a & b if spec[0] == "and" else a | b


def _draw(rng):
  while True:
    unit = rng.choice([16, 32, 128])
    sq = unit * rng.randint(1, 12)
    skv = sq if rng.random() < 0.5 else unit * rng.randint(1, 12)
    bq, bkv = unit * rng.choice([1, 1, 2, 4]), unit * rng.choice([1, 1, 2, 4])
    q_shards, kv_shards = rng.choice([1, 1, 2, 4]), rng.choice([1, 1, 2])
    if sq % bq or skv % bkv or (sq // bq) % q_shards or (skv // bkv) % kv_shards:
      continue
    spec = _leaf(rng, sq, skv)
    for _ in range(rng.choice([0, 0, 1, 2])):
      spec = (rng.choice(["and", "or"]), spec, _leaf(rng, sq, skv))
    return dict(sq=sq, skv=skv, block=(bq, bkv), spec=spec, dynamic_fwd=rng.random() < 0.7,
                dynamic_dkv=rng.random() < 0.5,
                kw=dict(downcast_smem_data=rng.random() < 0.7, q_seq_shards=q_shards, kv_seq_shards=kv_shards))


def _same(name, got, want, what):
  for field in FIELDS:
    a, b = got[field], want[field]
    assert (a is None) == (b is None), (name, field, what)
    if a is None:
      continue
    a, b = np.asarray(a), np.asarray(b)
    assert a.dtype == b.dtype and a.shape == b.shape, (name, field, a.dtype, b.dtype, a.shape, b.shape, what)
    assert np.array_equal(a, b), (name, field, what)


@pytest.mark.parametrize("seed", range(4))
def test_native_builder_agrees_with_the_restatement_on_random_masks(seed):
  ref = ref_loader.load_reference() if ref_loader.available() else None
  for case in range(40):
    c = _draw(random.Random(seed * 100003 + case))
    what = {k: v for k, v in c.items()}
    for is_dkv, dynamic in ((False, c["dynamic_fwd"]), (True, c["dynamic_dkv"])):
      mask = _make(c["spec"], mask_lib, c["sq"], c["skv"])
      fn = mask_info_lib.process_mask_dkv if is_dkv else mask_info_lib.process_mask
      try:
        native, _ = fn(mask, c["block"], return_dynamic_grid=dynamic, **c["kw"])
      except ValueError:
        with pytest.raises(ValueError):
          maskinfo_ref.process_mask(mask, c["block"], is_dkv, return_dynamic_grid=dynamic, **c["kw"])
        continue
      restated = maskinfo_ref.process_mask(mask, c["block"], is_dkv, return_dynamic_grid=dynamic, **c["kw"])
      _same("native vs restatement", native._asdict(), restated, what)
      if ref is not None:
        ref_mask, ref_mi = ref
        rfn = ref_mi.process_mask_dkv if is_dkv else ref_mi.process_mask
        theirs, _ = rfn(_make(c["spec"], ref_mask, c["sq"], c["skv"]), c["block"], return_dynamic_grid=dynamic, **c["kw"])
        _same("native vs reference", native._asdict(), theirs._asdict(), what)
