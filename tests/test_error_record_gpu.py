"""The device error record: a bounded wait that runs out, and what a raised record does.

Every device-side wait in the kernels is bounded; one that runs out writes the 4-word error record
and the kernel returns.  splash_probe_bounded_wait makes that happen on purpose in a one-thread
kernel (the wait gives up after a fraction of a millisecond), which is how the path is exercised
without hanging anything.
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


def test_bounded_wait_runs_out_and_is_reported():
  lib = _native.lib()
  err = torch.zeros(4, dtype=torch.int32, device=DEV)
  stream = C.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
  assert lib.splash_probe_bounded_wait(err.data_ptr(), 200000, 0x7e57, stream) == 0
  rec = (C.c_uint32 * 4)()
  st = lib.splash_read_error(err.data_ptr(), stream, C.byref(rec))
  assert st == -5, st  # SPLASH_ERR_KERNEL_TIMEOUT
  assert list(rec) == [1, 0, 0x7e57, 0]
  assert "bounded wait" in _native.status_str(st)
  # limits outside (0, 1e8] cycles are refused: the probe is not a way to stall a GPU
  assert lib.splash_probe_bounded_wait(err.data_ptr(), 0, 1, stream) == -1
  assert lib.splash_probe_bounded_wait(err.data_ptr(), 10**9, 1, stream) == -1
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
