"""Masks that are tensors on the device: schedules built there, no host round trip.

`make_dynamic_splash_mha(mask_on_gpu)` must give the result of the static path on the same mask
(bit for bit: the same tiles are visited in the same order, and partial tiles read the same mask
bytes), and the device-built tile states must equal a numpy classification.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref
from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
D = 128
DEV = "cuda:0"
SCALE = 1 / math.sqrt(D)


def _mask(sq, skv, seed):
  """Random mask with empty, full and partial 128x128 tiles, no dead row."""
  rng = np.random.default_rng(seed)
  m = rng.random((sq, skv)) < 0.5
  kind = rng.integers(0, 3, size=(sq // 128, skv // 128))
  for i in range(sq // 128):
    for j in range(skv // 128):
      if kind[i, j] == 0:
        m[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128] = False
      elif kind[i, j] == 2:
        m[i * 128:(i + 1) * 128, j * 128:(j + 1) * 128] = True
  m[np.arange(sq), np.arange(sq) % skv] = True
  return m


def test_tile_states_and_schedules_match_numpy():
  sq, skv = 640, 896
  m = _mask(sq, skv, 1)
  lib = _native.lib()
  md = torch.from_numpy(m).to(DEV)
  tables = splash._DynamicDeviceTables(md, batch=3)  # pylint: disable=protected-access
  torch.cuda.synchronize()
  blocks = m.reshape(sq // 128, 128, skv // 128, 128).swapaxes(1, 2)
  want = blocks.any(axis=(-1, -2)).astype(np.int32) + blocks.all(axis=(-1, -2)).astype(np.int32)
  np.testing.assert_array_equal(tables.tile_states.cpu().numpy(), want)
  nq, nkv = want.shape
  for kind, sched in ((0, tables.fwd), (1, tables.dq), (2, tables.dkv)):
    n_rows = sched.n_rows
    n_cols = nq if kind == 2 else nkv
    nbytes = lib.splash_dynamic_schedule_bytes(sq, skv, kind, 3)
    ws = next(t for t in tables.keep if t.dtype == torch.uint8 and t.numel() == nbytes and t.data_ptr() == sched.row_ptr)
    raw = ws.cpu().numpy()
    a256 = lambda n: (n + 255) & ~255
    row_ptr = raw[:4 * (n_rows + 1)].view(np.int32)
    off = a256(4 * (n_rows + 1))
    row_end = raw[off:off + 4 * 3 * n_rows].view(np.int32).reshape(3, n_rows)
    off += a256(4 * 3 * n_rows)
    entries = raw[off:off + 16 * n_rows * n_cols].view(np.int32).reshape(n_rows, n_cols, 4)
    np.testing.assert_array_equal(row_ptr, np.arange(n_rows + 1) * n_cols)
    for r in range(n_rows):
      if kind == 0:
        s0 = want[2 * r]
        s1 = want[2 * r + 1] if 2 * r + 1 < nq else np.zeros(nkv, np.int32)
      elif kind == 1:
        s0, s1 = want[r], np.zeros(nkv, np.int32)
      else:
        s0, s1 = want[:, r], np.zeros(nq, np.int32)
      live = np.nonzero(s0 | s1)[0]
      expect = np.stack([live, s0[live] | (s1[live] << 2), np.where(s0[live] == 1, 0, -1),
                         np.where(s1[live] == 1, 0, -1)], axis=1)
      assert (row_end[:, r] == r * n_cols + len(live)).all()
      np.testing.assert_array_equal(entries[r, :len(live)], expect)


@pytest.mark.parametrize("repeatable_dq", [True, False])
@pytest.mark.parametrize("with_segments", [False, True])
def test_device_mask_equals_static_path_bitwise(with_segments, repeatable_dq):
  b, hq, hkv, sq, skv = 2, 4, 2, 512, 768
  m = _mask(sq, skv, 2)
  g = torch.Generator().manual_seed(5)
  mk = lambda h, s: torch.randn(b, h, s, D, generator=g).to(torch.bfloat16).to(DEV)
  q, k, v, do = mk(hq, sq), mk(hkv, skv), mk(hkv, skv), mk(hq, sq)
  seg = None
  if with_segments:
    ids_q = torch.from_numpy(np.repeat(np.arange(4, dtype=np.int32), sq // 4))[None].expand(b, -1)
    ids_kv = torch.from_numpy(np.repeat(np.arange(4, dtype=np.int32), skv // 4))[None].expand(b, -1)
    seg = splash.SegmentIds(ids_q.to(DEV), ids_kv.to(DEV))
  results = []
  kw = dict(save_residuals=True, repeatable_dq=repeatable_dq)
  for kernel in (splash.make_dynamic_splash_mha(torch.from_numpy(m).to(DEV), **kw),
                 splash.make_splash_mha_single_device(mask_lib.NumpyMask(m), **kw)):
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    out, res = kernel(qa, ka, va, seg, logits_scale=SCALE)
    out.backward(do)
    kernel.check_errors()
    results.append((out, res["logsumexp"], qa.grad, ka.grad, va.grad))
  for i, (got, ref) in enumerate(zip(*results)):
    if i == 2 and not repeatable_dq:  # fused backward: dq is an fp32 sum in varying order
      assert ((got.float() - ref.float()).norm() / ref.float().norm()).item() <= 1e-3
    else:
      assert torch.equal(got, ref)
  if not with_segments:
    ro, rlse, _, rdq, rdk, rdv = attention_ref.fwd_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), m, None, scale=SCALE)
    out, lse, dq, dk, dv = results[0]
    assert ((out.float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
    assert (lse.cpu() - rlse).abs().max() <= 1e-3
    rel = lambda a, r: ((a.float().cpu() - r).norm() / r.norm()).item()
    assert rel(dq, rdq) <= 1e-2 and rel(dk, rdk) <= 1e-2 and rel(dv, rdv) <= 1e-2


def test_device_mask_info_is_available_on_request_and_bad_masks_are_rejected():
  m = _mask(256, 256, 3)
  kernel = splash.make_dynamic_splash_mha(torch.from_numpy(m).to(DEV))
  host = splash.make_dynamic_splash_mha(m)
  for a, b in zip(kernel.fwd_mask_info, host.fwd_mask_info):
    assert (a is None) == (b is None)
    if a is not None:
      np.testing.assert_array_equal(np.asarray(a), np.asarray(b))
  lib = _native.lib()
  assert lib.splash_mask_tile_states(None, 256, 256, 256, None, None) == -1
  assert lib.splash_dynamic_schedule_bytes(100, 256, 0, 1) == 0
  out = _native.SplashDeviceSchedule()
  assert lib.splash_dynamic_schedule(None, 256, 256, 0, 1, None, None, 0, C.byref(out), None) == -1
  with pytest.raises(ValueError):
    splash._DynamicDeviceTables(torch.zeros(256, 256, device=DEV), 1)  # pylint: disable=protected-access
