"""MaskInfo tables: oracle restatement and native builder vs tables made by the reference itself.

tests/golden/maskinfo_golden.npz was produced by the reference's own ``process_mask`` /
``process_mask_dkv`` (see tests/golden/gen_maskinfo_golden.py).  Everything is compared exactly:
values, dtypes, shapes, and which fields are None.
"""
import hashlib
import json
import os

import numpy as np
import pytest

import maskinfo_cases as cases
from oracle import maskinfo_ref
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import splash_attention_mask_info as mask_info_lib

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "maskinfo_golden.npz"))
NONE_FIELDS = set(json.loads(str(GOLDEN["__none__"])))
META = json.loads(str(GOLDEN["__meta__"]))


def _digest(a):
  h = hashlib.sha256()
  h.update(str(a.dtype).encode())
  h.update(str(a.shape).encode())
  h.update(np.ascontiguousarray(a).tobytes())
  return np.frombuffer(h.digest(), dtype=np.uint8)


def _check(case, tag, fields):
  for field in cases.FIELDS:
    key = f"{case['name']}/{tag}/{field}"
    got = fields[field]
    if key in NONE_FIELDS:
      assert got is None, f"{key}: expected None"
      continue
    assert got is not None, f"{key}: unexpectedly None"
    want = GOLDEN[key]
    got = np.asarray(got)
    if case["digest"]:
      assert np.array_equal(_digest(got), want), f"{key}: digest differs (dtype {got.dtype}, shape {got.shape})"
    else:
      assert got.dtype == want.dtype, f"{key}: dtype {got.dtype} != {want.dtype}"
      assert got.shape == want.shape, f"{key}: shape {got.shape} != {want.shape}"
      np.testing.assert_array_equal(got, want, err_msg=key)


def _kw(case):
  return dict(downcast_smem_data=case["downcast"], q_seq_shards=case["q_shards"], kv_seq_shards=case["kv_shards"])


def _q_len(spec):
  return spec[1] if isinstance(spec[1], int) else _q_len(spec[1])


# The restatement materialises every block like the reference, so it is kept to sizes it
# finishes in seconds.
ORACLE_CASES = [c for c in cases.CASES if _q_len(c["mask"]) <= 8192]


@pytest.mark.parametrize("case", ORACLE_CASES, ids=lambda c: c["name"])
def test_oracle_restatement_matches_reference_tables(case):
  mask = cases.build_mask(case["mask"], mask_lib)
  fwd = maskinfo_ref.process_mask(mask, tuple(case["block"]), False, **_kw(case))
  dkv = maskinfo_ref.process_mask(mask, tuple(case["block"]), True, return_dynamic_grid=case["dkv_dynamic"],
                                  **_kw(case))
  _check(case, "fwd", fwd)
  _check(case, "dkv", dkv)


@pytest.mark.parametrize("case", cases.CASES, ids=lambda c: c["name"])
def test_native_builder_matches_reference_tables(case):
  mask = cases.build_mask(case["mask"], mask_lib)
  fwd, fn = mask_info_lib.process_mask(mask, tuple(case["block"]), **_kw(case))
  dkv, fn2 = mask_info_lib.process_mask_dkv(mask, tuple(case["block"]),
                                            return_dynamic_grid=case["dkv_dynamic"], **_kw(case))
  assert (fn is not None) == META[case["name"]]["has_mask_function"]
  assert (fn is None) == (fn2 is None)
  _check(case, "fwd", fwd._asdict())
  _check(case, "dkv", dkv._asdict())
