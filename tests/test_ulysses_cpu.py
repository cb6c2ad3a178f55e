"""Ulysses exchange on CPU ranks (gloo, world_size 2): sharded == unsharded, forward and backward.

The attention inside is the CPU oracle (tests may use it); what is under test is the exchange,
its autograd and the segment-id gather — the host-side logic of the context-parallel path.
"""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_ref
from tokamax_b200 import base
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import ulysses


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _oracle_attention(mask_dense):
  """Differentiable fp32 attention over [B, H, S, D] built from the oracle's forward."""
  def fn(q, k, v, segment_ids, *, logits_scale):
    outs = []
    for b in range(q.shape[0]):
      seg = None if segment_ids is None else (segment_ids.q[b], segment_ids.kv[b])
      o, _, _ = attention_ref.attention_reference(q[b], k[b], v[b], mask_dense, seg, scale=logits_scale)
      outs.append(o)
    return torch.stack(outs)
  return fn


def _worker(rank, world, port, with_segments, result_queue, heads=(4, 2), batch=2):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    torch.manual_seed(0)
    (hq, hkv), b, s, d = heads, batch, 64, 16
    q = torch.randn(b, hq, s, d, requires_grad=True)
    k = torch.randn(b, hkv, s, d, requires_grad=True)
    v = torch.randn(b, hkv, s, d, requires_grad=True)
    do = torch.randn(b, hq, s, d)
    mask = mask_lib.make_causal_mask((s, s))
    seg = None
    if with_segments:
      ids = torch.from_numpy(np.repeat(np.arange(4, dtype=np.int32), s // 4))[None].expand(b, -1).contiguous()
      seg = base.SegmentIds(ids, ids)
    scale = 1 / math.sqrt(d)
    attn = _oracle_attention(mask)
    full = attn(q, k, v, seg, logits_scale=scale)
    full.backward(do)
    want = (full.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone())

    sl = slice(rank * s // world, (rank + 1) * s // world)
    ql, kl, vl = (t.detach()[:, :, sl].clone().requires_grad_(True) for t in (q, k, v))
    seg_l = None if seg is None else base.SegmentIds(seg.q[:, sl], seg.kv[:, sl])
    cp = ulysses.UlyssesSplashAttention(attn)
    out = cp(ql, kl, vl, seg_l, logits_scale=scale)
    out.backward(do[:, :, sl])
    got = (out.detach(), ql.grad, kl.grad, vl.grad)
    for g, w in zip(got, want):
      torch.testing.assert_close(g, w[:, :, sl], rtol=1e-5, atol=1e-5)
    # the exchange itself is exact and invertible
    x = torch.arange(b * hq * (s // world) * d, dtype=torch.float32).view(b, hq, s // world, d) + 1000 * rank
    y = ulysses.seq_to_head(x)
    assert y.shape == (b, hq // world, s, d)
    assert torch.equal(ulysses.head_to_seq(y), x)
    for src in range(world):
      expect = torch.arange(b * hq * (s // world) * d, dtype=torch.float32).view(b, hq, s // world, d) + 1000 * src
      blk = y[:, :, src * s // world:(src + 1) * s // world]
      assert torch.equal(blk, expect[:, rank * hq // world:(rank + 1) * hq // world])
    result_queue.put((rank, "ok"))
  except Exception as e:  # pylint: disable=broad-except
    result_queue.put((rank, f"{type(e).__name__}: {e}"))
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("with_segments", [False, True])
def test_ulysses_matches_unsharded_on_two_gloo_ranks(with_segments):
  world = 2
  ctx = mp.get_context("spawn")
  queue = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, with_segments, queue)) for r in range(world)]
  for p in procs:
    p.start()
  results = [queue.get(timeout=180) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
  assert sorted(results) == [(0, "ok"), (1, "ok")], results


@pytest.mark.parametrize("world,heads,batch", [(2, (4, 1), 1), (4, (8, 2), 2)])
def test_ulysses_replicates_kv_heads_when_ranks_outnumber_them(world, heads, batch):
  """More ranks than kv heads (MQA on 2 ranks; 2 kv heads on 4 ranks): the kv head a rank's q heads
  read is replicated to it, and its gradient is the sum over the copies."""
  ctx = mp.get_context("spawn")
  queue = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, False, queue, heads, batch)) for r in range(world)]
  for p in procs:
    p.start()
  results = [queue.get(timeout=180) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
  assert sorted(results) == [(r, "ok") for r in range(world)], results


def test_kv_head_assignment():
  f = ulysses.UlyssesSplashAttention.kv_heads_for_ranks
  assert f(64, 8, 8) is None and f(32, 8, 4) is None
  assert f(64, 8, 16) == [r // 2 for r in range(16)]
  assert f(8, 1, 4) == [0, 0, 0, 0]
  with pytest.raises(NotImplementedError):
    f(12, 4, 8)   # ranks do not divide the q heads
  assert f(12, 2, 4) == [0, 0, 1, 1]  # 3 q heads per rank, groups of 6
  with pytest.raises(NotImplementedError):
    f(12, 3, 2)   # 6 q heads per rank over groups of 4: a rank would straddle kv heads


def test_heads_not_divisible_is_rejected():
  class FakeGroup:
    pass
  # world size 1 never exchanges, so any head count passes through
  os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
  os.environ["MASTER_PORT"] = str(_free_port())
  dist.init_process_group("gloo", rank=0, world_size=1)
  try:
    x = torch.randn(1, 3, 8, 4)
    assert torch.equal(ulysses.seq_to_head(x), x)
    assert ulysses.exchange_bytes_sent((1, 8, 16, 128), 2, 8) == 1 * 8 * 16 * 128 * 2 * 7 // 8
  finally:
    dist.destroy_process_group()
