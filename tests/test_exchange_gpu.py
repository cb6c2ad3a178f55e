"""splash_exchange_push on one GPU: P ranks emulated by P calls whose destination pointers all lie
in this GPU's memory (the kernel only ever sees pointers, so the index arithmetic of every rank is
exercised without a second device).  Both directions, against the permutation written in torch."""
import ctypes as C

import pytest
import torch

from tokamax_b200 import _native

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


BASE = 4096  # the receive buffers sit this far inside their blocks (dst_base_bytes)


def _push(src, dst_bufs, rank, seq_to_head, batch, h_loc, s_loc, d):
  lib = _native.lib()
  ptrs = torch.tensor([t.data_ptr() - BASE for t in dst_bufs], dtype=torch.int64, device=DEV)
  a = _native.SplashExchangeArgs()
  a.src, a.dst_ptrs = src.data_ptr(), ptrs.data_ptr()
  a.world, a.rank, a.seq_to_head = len(dst_bufs), rank, int(seq_to_head)
  a.batch, a.h_loc, a.s_loc, a.row_bytes = batch, h_loc, s_loc, d * src.element_size()
  a.dst_base_bytes = BASE
  stream = C.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
  _native.check(lib.splash_exchange_push(C.byref(a), stream), "splash_exchange_push")
  torch.cuda.synchronize()


@pytest.mark.parametrize("world,batch,h_loc,s_loc,d", [(2, 1, 3, 256, 128), (4, 2, 2, 640, 64), (8, 1, 1, 384, 128)])
def test_exchange_push_both_directions(world, batch, h_loc, s_loc, d):
  heads, seq = h_loc * world, s_loc * world
  g = torch.Generator(device=DEV).manual_seed(world)
  full = torch.randn(batch, heads, seq, d, generator=g, device=DEV).to(torch.bfloat16)  # the unsharded tensor
  # sequence shards of all heads -> head shards of the whole sequence
  head_bufs = [torch.zeros(batch, h_loc, seq, d, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
  for r in range(world):
    src = full[:, :, r * s_loc:(r + 1) * s_loc].contiguous()
    _push(src, head_bufs, r, True, batch, h_loc, s_loc, d)
  for j in range(world):
    assert torch.equal(head_bufs[j], full[:, j * h_loc:(j + 1) * h_loc])
  # and back
  seq_bufs = [torch.zeros(batch, heads, s_loc, d, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
  for r in range(world):
    _push(head_bufs[r], seq_bufs, r, False, batch, h_loc, s_loc, d)
  for j in range(world):
    assert torch.equal(seq_bufs[j], full[:, :, j * s_loc:(j + 1) * s_loc])


def test_exchange_push_rejects_bad_arguments():
  lib = _native.lib()
  assert lib.splash_exchange_push(None, None) == -1
  a = _native.SplashExchangeArgs()
  x = torch.zeros(1, 2, 128, 128, dtype=torch.bfloat16, device=DEV)
  ptrs = torch.tensor([x.data_ptr(), x.data_ptr()], dtype=torch.int64, device=DEV)
  a.src, a.dst_ptrs, a.world, a.rank, a.seq_to_head = x.data_ptr(), ptrs.data_ptr(), 2, 2, 1
  a.batch, a.h_loc, a.s_loc, a.row_bytes = 1, 1, 128, 256
  assert lib.splash_exchange_push(C.byref(a), None) == -1  # rank out of range
  a.rank, a.row_bytes = 0, 250
  assert lib.splash_exchange_push(C.byref(a), None) == -1  # rows not a multiple of 16 bytes
