"""Ring attention on CPU ranks (gloo): sharded == unsharded, forward and backward.

The per-pair attention inside is the CPU oracle (tests may use it); under test are the sub-mask
construction, the rotation of key / value shards, the logsumexp merge, and the dk / dv
accumulators travelling with their shard — the host-side logic of the ring.
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
from tokamax_b200 import ring_attention as ring
from tokamax_b200 import splash_attention_mask as mask_lib


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


class OracleShard:
  """`ShardAttention` built from the oracle: one (query shard, key shard) pair."""

  def __init__(self, sub_mask):
    self.dense = np.asarray(sub_mask[:, :]).astype(bool)
    self.empty = not self.dense.any()

  def forward(self, q, k, v, q_seg, kv_seg, scale):
    outs, lses = [], []
    for b in range(q.shape[0]):
      seg = None if q_seg is None else (q_seg[b], kv_seg[b])
      o, lse, _ = attention_ref.attention_reference(q[b], k[b], v[b], self.dense, seg, scale=scale)
      outs.append(o)
      lses.append(lse)
    return torch.stack(outs), torch.stack(lses)

  def backward(self, q, k, v, o, lse, d_o, q_seg, kv_seg, scale):
    grads = []
    for b in range(q.shape[0]):
      seg = None if q_seg is None else (q_seg[b], kv_seg[b])
      grads.append(attention_ref.attention_reference_vjp(d_o[b], q[b], k[b], v[b], self.dense, seg, o[b], lse[b],
                                                         scale=scale))
    return tuple(torch.stack([g[i] for g in grads]) for i in range(3))


def _mask(kind, s):
  if kind == "causal":
    return mask_lib.CausalMask((s, s))
  if kind == "local":
    return mask_lib.LocalMask((s, s), (s // 3, 5), 0)
  if kind == "chunked":
    return mask_lib.ChunkedCausalMask((s, s), s // 6)
  if kind == "composed":
    return mask_lib.LogicalAnd(mask_lib.LocalMask((s, s), (s // 2, None), 0), mask_lib.CausalMask((s, s)))
  return mask_lib.NumpyMask(mask_lib.make_random_mask((s, s), 0.5, 7) | np.eye(s, dtype=bool))


def _worker(rank, world, port, kind, with_segments, queue, layout="contiguous"):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    torch.manual_seed(0)
    b, hq, hkv, s, d = 2, 3, 1, 48 * world, 16  # 3 q heads on 2 ranks: no divisibility needed
    q = torch.randn(b, hq, s, d)
    k = torch.randn(b, hkv, s, d)
    v = torch.randn(b, hkv, s, d)
    do = torch.randn(b, hq, s, d)
    mask = _mask(kind, s)
    dense = np.asarray(mask[:, :])
    seg = None
    if with_segments:
      ids = torch.from_numpy(np.repeat(np.arange(3, dtype=np.int32), s // 3))[None].expand(b, -1).contiguous()
      seg = (ids, ids)
    scale = 1 / math.sqrt(d)
    want = attention_ref.fwd_bwd(q, k, v, do, dense, seg, scale=scale)
    # fwd_bwd takes di from the output rounded to the input dtype; fp32 here, so nothing is rounded

    if layout == "zigzag":
      take = lambda t, dim=2: ring.zigzag_shard(t, rank, world, dim)
    else:
      take = lambda t, dim=2: t.narrow(dim, rank * s // world, s // world)
    ql, kl, vl = (take(t).clone().requires_grad_(True) for t in (q, k, v))
    seg_l = None if seg is None else base.SegmentIds(take(seg[0], 1), take(seg[1], 1))
    attn = ring.RingSplashAttention(mask, save_residuals=True, shard_attention_factory=OracleShard, layout=layout)
    out, res = attn(ql, kl, vl, seg_l, logits_scale=scale)
    out.backward(take(do))
    ro, rlse, _, rdq, rdk, rdv = want
    for got, ref in ((out.detach(), ro), (res["logsumexp"], rlse), (ql.grad, rdq), (kl.grad, rdk), (vl.grad, rdv)):
      torch.testing.assert_close(got, take(ref), rtol=2e-5, atol=2e-5)
    if layout == "zigzag" and kind == "causal":  # every rank has the same number of live chunk pairs
      live = sum(not attn.pair_attention(a, c, world).empty
                 for a in attn.chunks_of(rank, world) for r2 in range(world) for c in attn.chunks_of(r2, world))
      assert live == 2 * world + 1
    # pairs above the causal diagonal are recognised as empty and skipped
    if kind == "causal" and world > 1 and layout == "contiguous":
      assert attn.shard_attention(0, world - 1).empty and not attn.shard_attention(world - 1, 0).empty
    queue.put((rank, "ok"))
  except Exception as e:  # pylint: disable=broad-except
    import traceback
    queue.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
  finally:
    dist.destroy_process_group()


def _run(world, kind, with_segments, layout="contiguous"):
  ctx = mp.get_context("spawn")
  queue = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, kind, with_segments, queue, layout))
           for r in range(world)]
  for p in procs:
    p.start()
  results = [queue.get(timeout=240) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
  assert sorted(results) == [(r, "ok") for r in range(world)], results


@pytest.mark.parametrize("kind,with_segments", [("causal", False), ("local", True), ("numpy", False)])
def test_ring_matches_unsharded_on_two_gloo_ranks(kind, with_segments):
  _run(2, kind, with_segments)


@pytest.mark.parametrize("kind", ["composed", "chunked"])
def test_ring_on_three_gloo_ranks(kind):
  _run(3, kind, kind == "composed")


@pytest.mark.parametrize("world,kind,with_segments", [(2, "causal", False), (3, "local", True), (2, "numpy", False)])
def test_zigzag_ring_matches_unsharded(world, kind, with_segments):
  _run(world, kind, with_segments, layout="zigzag")


def test_zigzag_shard_round_trip():
  x = torch.arange(2 * 3 * 24 * 2, dtype=torch.float32).view(2, 3, 24, 2)
  shards = [ring.zigzag_shard(x, r, 3) for r in range(3)]
  assert shards[0].shape == (2, 3, 8, 2)
  assert torch.equal(shards[1][:, :, :4], x[:, :, 4:8]) and torch.equal(shards[1][:, :, 4:], x[:, :, 16:20])
  assert torch.equal(ring.zigzag_unshard(shards), x)
  with pytest.raises(ValueError):
    ring.RingSplashAttention(mask_lib.FullMask((8, 8)), layout="spiral")


@pytest.mark.parametrize("kind", ["causal", "local", "chunked", "composed", "numpy"])
def test_shard_mask_is_the_window_of_the_mask(kind):
  s, shards = 96, 3
  mask = _mask(kind, s)
  dense = np.asarray(mask[:, :])
  n = s // shards
  for r in range(shards):
    for c in range(shards):
      sub = ring.shard_mask(mask, r, c, shards, shards)
      assert sub.shape == (n, n)
      np.testing.assert_array_equal(np.asarray(sub[:, :]), dense[r * n:(r + 1) * n, c * n:(c + 1) * n])
  # lazy masks stay lazy (no O(S^2) array is built for them)
  if kind in ("causal", "local"):
    assert not isinstance(ring.shard_mask(mask, 2, 0, shards, shards), mask_lib.NumpyMask)
  with pytest.raises(ValueError):
    ring.shard_mask(mask, 0, 0, 5, 5)


def test_merge_partial_is_a_logsumexp_weighted_mean():
  g = torch.Generator().manual_seed(1)
  o1, o2 = torch.randn(2, 3, 8, 4, generator=g), torch.randn(2, 3, 8, 4, generator=g)
  l1, l2 = torch.randn(2, 3, 8, generator=g), torch.randn(2, 3, 8, generator=g)
  l2[0, 0, :2] = -2.0e38  # rows with no live key on the second shard
  o_acc = torch.zeros_like(o1)
  lse_acc = torch.full_like(l1, -float("inf"))
  ring.merge_partial(o_acc, lse_acc, o1, l1)
  ring.merge_partial(o_acc, lse_acc, o2, l2)
  w1, w2 = torch.exp(l1.double()), torch.exp(l2.double())
  want = (o1.double() * w1[..., None] + o2.double() * w2[..., None]) / (w1 + w2)[..., None]
  torch.testing.assert_close(o_acc.double(), want, rtol=1e-5, atol=1e-6)
  torch.testing.assert_close(lse_acc.double(), torch.log(w1 + w2), rtol=1e-5, atol=1e-6)
  assert torch.equal(o_acc[0, 0, :2], o1[0, 0, :2])
