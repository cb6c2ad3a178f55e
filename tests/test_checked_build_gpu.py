"""The "checked" build of the library against the default build, and the device error record.

The default build's MMA-issuing threads go from an mbarrier wait straight to the tcgen05.mma that
consumes what the wait published (TMEM written by other warps' tcgen05.st, fenced and completed on
the producer side); the checked build puts a tcgen05.fence::after_thread_sync in between, as the
PTX ordering rules ask.  Both must give the same bits.  The checked build also exports a probe
kernel whose bounded wait runs out, which is how the error path is exercised without hanging
anything: the wait gives up after a fraction of a millisecond and the kernel returns.
"""
import ctypes as C
import math

import pytest
import torch

import abi_util
from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
D = 128
DEV = torch.device("cuda:0")
SCALE = 1 / math.sqrt(D)


def _inputs(seed, b, hq, hkv, s):
  g = torch.Generator().manual_seed(seed)
  mk = lambda h: torch.randn(b, h, s, D, generator=g).to(torch.bfloat16).to(DEV)
  return mk(hq), mk(hkv), mk(hkv), mk(hq)


@pytest.mark.parametrize("mask_kind", ["causal", "local"])
def test_fenced_issue_path_gives_the_same_bits(mask_kind):
  """Forward, dq, dkv (split form) bit for bit; fused form: o, lse, dk, dv bit for bit."""
  s = 1024
  mask = mask_lib.CausalMask((s, s)) if mask_kind == "causal" else mask_lib.LocalMask((s, s), (200, 100), 0)
  kernel = splash.make_splash_mha(mask, q_seq_shards=1)
  q, k, v, do = _inputs(41, 2, 8, 8 if mask_kind == "causal" else 2, s)
  default, checked = _native.lib(), _native.lib_variant("checked")
  for fused in (False, True):
    a = abi_util.fwd_bwd(default, kernel, q, k, v, do, SCALE, fused=fused)
    b = abi_util.fwd_bwd(checked, kernel, q, k, v, do, SCALE, fused=fused)
    kernel.check_errors()
    for name, x, y in zip(("o", "lse", "dq", "dk", "dv"), a, b):
      if fused and name == "dq":
        assert ((x.float() - y.float()).norm() / y.float().norm()).item() <= 1e-3
      else:
        assert torch.equal(x, y), (name, fused)


def test_bounded_wait_runs_out_and_is_reported():
  lib = _native.lib_variant("checked")
  err = torch.zeros(4, dtype=torch.int32, device=DEV)
  stream = C.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
  assert lib.splash_test_bounded_wait(err.data_ptr(), 200000, 0x7e57, stream) == 0
  rec = (C.c_uint32 * 4)()
  st = lib.splash_read_error(err.data_ptr(), stream, C.byref(rec))
  assert st == -5, st  # SPLASH_ERR_KERNEL_TIMEOUT
  assert list(rec) == [1, 0, 0x7e57, 0]
  assert "bounded wait" in _native.status_str(st)
  # limits outside (0, 1e8] cycles are refused: the probe is not a way to stall a GPU
  assert lib.splash_test_bounded_wait(err.data_ptr(), 0, 1, stream) == -1
  assert lib.splash_test_bounded_wait(err.data_ptr(), 10**9, 1, stream) == -1
  # the context is still usable
  assert torch.ones(8, device=DEV).sum().item() == 8


def test_a_raised_error_record_stops_later_kernels_and_check_errors_clears_it():
  """Once a record holds an error every kernel given that record returns at once and leaves its
  outputs alone; check_errors() raises, clears the record, and the kernel object works again."""
  s = 512
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  q, k, v, do = _inputs(43, 1, 4, 2, s)
  tables = kernel._tables(DEV, 1)  # pylint: disable=protected-access
  tables.error_record[0] = 1
  tables.error_record[2] = 0x1234
  for fused in (False, True):
    o, lse, dq, dk, dv = abi_util.fwd_bwd(_native.lib(), kernel, q, k, v, do, SCALE, fused=fused, fill=7.0)
    for name, t in (("o", o), ("lse", lse), ("dk", dk), ("dv", dv)):
      assert (t == 7.0).all(), name
    if not fused:  # (the fused form's cast pass is not an attention kernel; it writes the zeroed image)
      assert (dq == 7.0).all()
  with pytest.raises(_native.SplashError) as exc:
    kernel.check_errors()
  assert exc.value.status == -5 and "4660" in str(exc.value)
  kernel.check_errors()  # cleared
  qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
  out = kernel(qd, kd, vd, logits_scale=SCALE)
  out.backward(do)
  kernel.check_errors()
  assert torch.isfinite(out.float()).all() and torch.isfinite(qd.grad.float()).all()
