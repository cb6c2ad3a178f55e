"""The backward entry point that brings its own scratch (splash_bwd_static_scratch).

Some callers of the backward pass cannot hand it a workspace: a custom-call handler that only
receives the operand and result buffers its runtime chose, or code that runs where entering an
allocator is not possible.  For them the library keeps the scratch (the per-row terms di and
-logsumexp*log2e) in an array inside its own image, at most SPLASH_STATIC_SCRATCH_MAX_ROWS rows.
This test calls that entry point through the C ABI and checks dQ / dK / dV against the regular
splash_bwd (caller-provided workspace) on two calls in a row with different inputs — the second
call sees the first call's leftovers in the shared array and must not be affected by them.
Kernels and arithmetic are the same on both paths, so results are compared bit for bit.
The file name keeps it last in collection order.
"""
import ctypes as C
import math

import pytest
import torch

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
D = 128
MAX_ROWS = 1 << 20  # SPLASH_STATIC_SCRATCH_MAX_ROWS in include/splash_b200.h


def _backward_both_ways(kernel, seed, b, hq, hkv, s, dev):
  g = torch.Generator(device=dev).manual_seed(seed)
  mk = lambda h: torch.randn(b, h, s, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
  q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
  scale = 1 / math.sqrt(D)
  out, res = kernel(q, k, v, logits_scale=scale, save_residuals=True)
  lse = res["logsumexp"].contiguous()
  tables = kernel._tables(dev)  # pylint: disable=protected-access
  lib = _native.lib()
  stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

  def args_for(dq, dk, dv):
    a = _native.SplashBwdArgs()
    a.q, a.k, a.v, a.o, a.d_o = map(splash._tensor_desc, (q, k, v, out, do))  # pylint: disable=protected-access
    a.dq, a.dk, a.dv = map(splash._tensor_desc, (dq, dk, dv))  # pylint: disable=protected-access
    a.logsumexp = lse.data_ptr()
    a.sched_dq, a.sched_dkv = tables.dq, tables.dkv
    a.mask_fn = splash._mask_fn_struct(kernel.mask_function_rule)  # pylint: disable=protected-access
    a.scale = scale
    a.error_record = tables.error_record.data_ptr()
    return a

  ref = [torch.empty_like(t) for t in (q, k, v)]
  a = args_for(*ref)
  ws_bytes = lib.splash_bwd_workspace_bytes(b, hq, s)
  ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
  a.workspace, a.workspace_bytes = ws.data_ptr(), ws_bytes
  _native.check(lib.splash_bwd(C.byref(a), stream), "splash_bwd")

  got = [torch.full_like(t, float("nan")) for t in (q, k, v)]
  a2 = args_for(*got)  # workspace left NULL on purpose: this entry point must not need one
  _native.check(lib.splash_bwd_static_scratch(C.byref(a2), stream), "splash_bwd_static_scratch")
  torch.cuda.synchronize(dev)
  kernel.check_errors()
  return ref, got


def test_static_scratch_backward_matches_regular_backward_twice_in_a_row():
  dev = torch.device("cuda:0")
  s = 1024
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  for seed, (b, hq, hkv) in ((1, (2, 8, 2)), (2, (1, 4, 4))):
    ref, got = _backward_both_ways(kernel, seed, b, hq, hkv, s, dev)
    for name, r, g in zip(("dq", "dk", "dv"), ref, got):
      assert torch.isfinite(g.float()).all(), name
      assert torch.equal(r, g), f"{name} differs on call with seed {seed}"


def test_static_scratch_backward_rejects_sizes_beyond_its_limit():
  dev = torch.device("cuda:0")
  lib = _native.lib()
  s = 1024
  b, hq = 2, (MAX_ROWS // s) // 2 + 1  # one head too many: b * hq * s > MAX_ROWS
  a = _native.SplashBwdArgs()
  for t in (a.q, a.o, a.d_o, a.dq):
    t.size[0], t.size[1], t.size[2], t.size[3] = b, hq, s, D
  st = lib.splash_bwd_static_scratch(C.byref(a), None)
  assert st == -7, st  # SPLASH_ERR_TOO_LARGE, before any launch or pointer is touched
  assert "SPLASH_STATIC_SCRATCH_MAX_ROWS" in lib.splash_status_str(st).decode()
  assert lib.splash_bwd_static_scratch(None, None) == -1
