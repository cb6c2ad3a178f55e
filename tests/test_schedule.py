"""Kernel schedule builder vs a brute-force expansion, and MaskInfo -> block-grid round trips."""
import ctypes as C

import numpy as np
import pytest

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import splash_attention_mask_info as mi


def _build(state, pid, bq, bkv, kind):
  out = _native.SplashScheduleOut()
  lib = _native.lib()
  state = np.ascontiguousarray(state, np.int32)
  pid = np.ascontiguousarray(pid, np.int32)
  _native.check(lib.splash_schedule_build(state.ctypes.data, pid.ctypes.data, state.shape[0], state.shape[1],
                                          bq, bkv, kind, C.byref(out)), "schedule")
  rp = np.ctypeslib.as_array(out.row_ptr, shape=(out.n_rows + 1,)).copy()
  en = np.ctypeslib.as_array(out.entries, shape=(max(out.n_entries, 1), 4)).copy()[:out.n_entries]
  order = np.ctypeslib.as_array(out.row_order, shape=(out.n_rows,)).copy()
  lib.splash_schedule_free(C.byref(out))
  # launch order: a permutation of the rows, longest first, ties by row index
  counts = np.diff(rp)
  np.testing.assert_array_equal(order, np.argsort(-counts, kind="stable"))
  return rp, en


def _brute(state, pid, bq, bkv, kind):
  fq, fkv = bq // 128, bkv // 128
  tq, tkv = state.shape[0] * fq, state.shape[1] * fkv
  st = lambda q, k: int(state[q // fq, k // fkv])
  pd = lambda q, k: int(pid[q // fq, k // fkv])
  rows = []
  if kind == 0:
    for r in range((tq + 1) // 2):
      ents = []
      for k in range(tkv):
        s0 = st(2 * r, k)
        s1 = st(2 * r + 1, k) if 2 * r + 1 < tq else 0
        if s0 or s1:
          ents.append([k, s0 | (s1 << 2), pd(2 * r, k) if s0 == 1 else -1, pd(2 * r + 1, k) if s1 == 1 else -1])
      rows.append(ents)
  elif kind == 1:
    for q in range(tq):
      rows.append([[k, st(q, k), pd(q, k) if st(q, k) == 1 else -1, -1] for k in range(tkv) if st(q, k)])
  else:
    for k in range(tkv):
      rows.append([[q, st(q, k), pd(q, k) if st(q, k) == 1 else -1, -1] for q in range(tq) if st(q, k)])
  rp = np.cumsum([0] + [len(r) for r in rows]).astype(np.int32)
  en = np.array([e for r in rows for e in r], np.int32).reshape(-1, 4)
  return rp, en


@pytest.mark.parametrize("kind", [0, 1, 2])
@pytest.mark.parametrize("bq,bkv,nq,nkv", [(128, 128, 5, 7), (256, 128, 3, 4), (128, 512, 6, 2), (512, 256, 2, 3)])
def test_schedule_matches_brute_force(kind, bq, bkv, nq, nkv):
  rng = np.random.default_rng(kind * 100 + nq * 10 + nkv)
  state = rng.integers(0, 3, size=(nq, nkv)).astype(np.int32)
  pid = np.where(state == 1, rng.integers(0, 9, size=(nq, nkv)), -1).astype(np.int32)
  rp, en = _build(state, pid, bq, bkv, kind)
  brp, ben = _brute(state, pid, bq, bkv, kind)
  np.testing.assert_array_equal(rp, brp)
  np.testing.assert_array_equal(en, ben)


def test_empty_rows_and_all_empty_mask():
  state = np.zeros((3, 3), np.int32)
  pid = np.full((3, 3), -1, np.int32)
  for kind, n_rows in ((0, 2), (1, 3), (2, 3)):
    rp, en = _build(state, pid, 128, 128, kind)
    assert list(rp) == [0] * (n_rows + 1) and en.shape[0] == 0


@pytest.mark.parametrize("dyn", [True, False])
def test_block_grids_round_trip(dyn):
  s = 1024
  mask = mask_lib.LocalMask((s, s), (300, None), 0) & mask_lib.CausalMask((s, s))
  dense = np.asarray(mask[(slice(0, s), slice(0, s))])
  blocks = dense.reshape(8, 128, 8, 128).swapaxes(1, 2)
  want = blocks.any((-1, -2)).astype(np.int32) + blocks.all((-1, -2)).astype(np.int32)
  fwd, _ = mi.process_mask(mask, (128, 128))
  dkv, _ = mi.process_mask_dkv(mask, (128, 128), return_dynamic_grid=dyn)
  for info, is_dkv in ((fwd, False), (dkv, True)):
    state, pid = mi.block_grids(info, 8, 8, is_dkv=is_dkv)
    np.testing.assert_array_equal(state, want)
    for (i, j) in zip(*np.nonzero(state == 1)):
      blk = info.partial_mask_blocks[pid[i, j]]
      blk = blk.T if is_dkv else blk
      np.testing.assert_array_equal(blk.astype(bool), blocks[i, j])
  full_state, full_pid = mi.block_grids(mi.process_mask(mask_lib.FullMask((256, 512)), (128, 128))[0], 2, 4, is_dkv=False)
  assert (full_state == 2).all() and (full_pid == -1).all()
