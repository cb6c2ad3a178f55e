"""Context parallelism for splash attention: the Ulysses sequence <-> head exchange.

Every rank holds a contiguous sequence shard of q, k, v (all heads).  An all-to-all turns that
into a head shard over the whole sequence, the unsharded splash kernel runs on the local heads
with the full-sequence MaskInfo (identical on every rank), and a second all-to-all brings the
output back to sequence shards.  The backward pass is the same two exchanges reversed, obtained
through autograd.

The reference has no all-to-all; its context-parallel wrapper is ring attention
(tokamax/_src/ops/experimental/tpu/splash_attention/ring_attention_kernel.py:68-293).  The
contract kept here is the one its tests state for sharded execution
(ring_attention_kernel_test.py:136-172): the sharded result equals the unsharded splash call on
the gathered inputs.  Because the kernels are deterministic and each rank computes whole heads,
the result is bitwise equal to a single-GPU run of the same heads.

Layout: tensors are ``[batch, heads, seq, head_dim]``.  The exchange posts one send and one
receive per (peer, batch, head) slab — a contiguous ``[seq/P, head_dim]`` block on both sides — so
data lands directly in the ``[batch, heads/P, seq, head_dim]`` layout the kernels read: there is
no pack or unpack copy on either side of the collective.  With NCCL the slabs of one exchange
are coalesced into a single group launch over NVLink.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from tokamax_b200 import base


def _world(group) -> tuple[int, int]:
  return dist.get_rank(group), dist.get_world_size(group)


def _exchange(x: torch.Tensor, group, seq_to_head: bool) -> torch.Tensor:
  """seq_to_head: [B, H, S/P, D] -> [B, H/P, S, D]; otherwise the inverse."""
  rank, world = _world(group)
  if world == 1:
    return x
  x = x.contiguous()
  b = x.shape[0]
  if seq_to_head:
    h_all, s_loc = x.shape[1], x.shape[2]
    if h_all % world != 0:
      raise ValueError(f"heads ({h_all}) must be divisible by the context-parallel size ({world})")
    h_loc = h_all // world
    out = torch.empty((b, h_loc, s_loc * world, x.shape[3]), dtype=x.dtype, device=x.device)
  else:
    h_loc, s_all = x.shape[1], x.shape[2]
    if s_all % world != 0:
      raise ValueError(f"sequence ({s_all}) must be divisible by the context-parallel size ({world})")
    s_loc = s_all // world
    out = torch.empty((b, h_loc * world, s_loc, x.shape[3]), dtype=x.dtype, device=x.device)

  ops = []
  for step in range(world):
    # stagger peers so that no rank is everybody's first target
    peer = (rank + step) % world
    for bi in range(b):
      for h in range(h_loc):
        if seq_to_head:
          send = x[bi, peer * h_loc + h]                              # my seq shard, peer's head
          recv = out[bi, h, peer * s_loc:(peer + 1) * s_loc]          # peer's seq shard, my head
        else:
          send = x[bi, h, peer * s_loc:(peer + 1) * s_loc]            # peer's seq shard, my head
          recv = out[bi, peer * h_loc + h]                            # my seq shard, peer's head
        if peer == rank:
          recv.copy_(send)
        else:
          ops.append(dist.P2POp(dist.isend, send, dist.get_global_rank(group, peer) if group else peer, group))
          ops.append(dist.P2POp(dist.irecv, recv, dist.get_global_rank(group, peer) if group else peer, group))
  if ops:
    for work in dist.batch_isend_irecv(ops):
      work.wait()
  return out


class _SeqToHead(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _exchange(x, group, True)

  @staticmethod
  def backward(ctx, g):
    return _exchange(g, ctx.group, False), None


class _HeadToSeq(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _exchange(x, group, False)

  @staticmethod
  def backward(ctx, g):
    return _exchange(g, ctx.group, True), None


def seq_to_head(x: torch.Tensor, group=None) -> torch.Tensor:
  """Differentiable all-to-all: sequence shard of all heads -> all of the sequence for H/P heads."""
  return _SeqToHead.apply(x, group)


def head_to_seq(x: torch.Tensor, group=None) -> torch.Tensor:
  """Differentiable inverse of :func:`seq_to_head`."""
  return _HeadToSeq.apply(x, group)


def exchange_bytes_sent(shape, itemsize: int, world: int) -> int:
  """Bytes one rank puts on the wire for one exchange of a local tensor of ``shape``."""
  n = itemsize
  for s in shape:
    n *= s
  return n * (world - 1) // world


class UlyssesSplashAttention:
  """Sequence-sharded splash attention.

  Args:
    attention: a ``SplashAttentionKernel`` built for the FULL (unsharded) mask, or any callable
      ``(q, k, v, segment_ids, *, logits_scale) -> out`` over ``[batch, heads, seq, dim]``.
    group: process group spanning the context-parallel ranks (default: the world).

  Call with the local sequence shards ``q [B, Hq, S/P, D]``, ``k, v [B, Hkv, S/P, D]``; rank ``r``
  holds tokens ``[r*S/P, (r+1)*S/P)``.  ``P`` must divide both head counts, which keeps the
  reference's GQA mapping ``kv_head = q_head // (Hq / Hkv)`` rank-local.  Returns the local
  sequence shard of the output ``[B, Hq, S/P, D]``.
  """

  def __init__(self, attention: Callable, group=None):
    self.attention = attention
    self.group = group

  def __call__(self, q, k, v, segment_ids: base.SegmentIds | None = None, *, logits_scale: float = 1.0):
    _, world = _world(self.group)
    if q.shape[1] % world != 0 or k.shape[1] % world != 0:
      raise NotImplementedError(
          f"context-parallel size {world} must divide q heads ({q.shape[1]}) and kv heads ({k.shape[1]}); "
          "kv-head replication is not built"
      )
    q_h = seq_to_head(q, self.group)
    k_h = seq_to_head(k, self.group)
    v_h = seq_to_head(v, self.group)
    seg_full = None
    if segment_ids is not None:
      seg_full = base.SegmentIds(self._gather_seq(segment_ids.q), self._gather_seq(segment_ids.kv))
    o_h = self.attention(q_h, k_h, v_h, seg_full, logits_scale=logits_scale)
    return head_to_seq(o_h, self.group)

  def _gather_seq(self, ids: torch.Tensor) -> torch.Tensor:
    _, world = _world(self.group)
    if world == 1:
      return ids
    ids = ids.contiguous()
    parts = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(parts, ids, group=self.group)
    return torch.cat(parts, dim=-1)
