"""Helpers for tests that call the kernels straight through the C ABI of a given library build."""
import ctypes as C

import torch

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as splash


def fwd_bwd(lib, kernel, q, k, v, do, scale, *, fused=False, error_record=None, fill=None):
  """splash_fwd then splash_bwd of `lib` on [B, H, S, 128] bf16 CUDA tensors.

  Returns (o, lse, dq, dk, dv).  `fill`: value the outputs hold before the calls (default: whatever
  torch.empty left there).  `error_record`: 4 x int32 device tensor (default: the kernel object's).
  """
  dev = q.device
  tables = kernel._tables(dev, q.shape[0])  # pylint: disable=protected-access
  err = tables.error_record if error_record is None else error_record
  b, hq, s, _ = q.shape
  mk = (lambda t: torch.empty_like(t)) if fill is None else (lambda t: torch.full_like(t, fill))
  o, dq, dk, dv = mk(q), mk(q), mk(k), mk(v)
  lse = torch.empty((b, hq, s), dtype=torch.float32, device=dev) if fill is None else \
      torch.full((b, hq, s), fill, dtype=torch.float32, device=dev)
  stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
  desc = splash._tensor_desc  # pylint: disable=protected-access
  fa = _native.SplashFwdArgs()
  fa.q, fa.k, fa.v, fa.o = map(desc, (q, k, v, o))
  fa.logsumexp = lse.data_ptr()
  fa.sched = tables.fwd
  fa.mask_fn = splash._mask_fn_struct(kernel.mask_function_rule)  # pylint: disable=protected-access
  fa.scale = scale
  fa.mask_value = -1e30
  fa.error_record = err.data_ptr()
  fa.q_sequence = tables.q_sequence.data_ptr() if tables.q_sequence is not None else None
  _native.check(lib.splash_fwd(C.byref(fa), stream), "splash_fwd")
  ba = _native.SplashBwdArgs()
  ba.q, ba.k, ba.v, ba.o, ba.d_o = map(desc, (q, k, v, o, do))
  ba.dq, ba.dk, ba.dv = map(desc, (dq, dk, dv))
  ba.logsumexp = lse.data_ptr()
  ba.sched_dq, ba.sched_dkv = tables.dq, tables.dkv
  ba.mask_fn = fa.mask_fn
  ba.q_sequence = fa.q_sequence
  ba.scale = scale
  ba.error_record = err.data_ptr()
  ba.flags = _native.BWD_FUSED_DQ if fused else 0
  size_fn = lib.splash_bwd_fused_workspace_bytes if fused else lib.splash_bwd_workspace_bytes
  ws_bytes = size_fn(b, hq, s)
  ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
  ba.workspace, ba.workspace_bytes = ws.data_ptr(), ws_bytes
  _native.check(lib.splash_bwd(C.byref(ba), stream), "splash_bwd")
  torch.cuda.synchronize(dev)
  return o, lse, dq, dk, dv
