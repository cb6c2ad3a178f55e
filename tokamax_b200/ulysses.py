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

Layout: tensors are ``[batch, heads, seq, head_dim]``.  An exchange is ONE collective
(``all_to_all_single``, which NCCL runs as a single grouped transfer over NVLink): the send buffer is
peer-major ``[P, batch, heads/P, seq/P, head_dim]`` — for ``batch == 1`` that is the tensor itself,
otherwise one permuting copy — and the receive buffer ``[P(source), batch, heads/P, seq/P, head_dim]``
is permuted into ``[batch, heads/P, seq, head_dim]`` (a view when one head arrives per rank, as for the
K / V of a GQA model whose kv-head count equals ``P``; one local copy otherwise).  The kernels then
read the result in place through their strided tensor maps.

When ``P`` does not divide the kv-head count but every rank's q heads share one kv head (``P`` a
multiple of ``Hkv``, e.g. 8 kv heads on 16 GPUs), that kv head is replicated: each rank receives the
whole sequence of the one kv head its q heads read, and the backward pass sums the gradients of the
copies (autograd of the head gather) after the reverse exchange.
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
  _, world = _world(group)
  if world == 1:
    return x
  b, d = x.shape[0], x.shape[3]
  if seq_to_head:
    h_all, s_loc = x.shape[1], x.shape[2]
    if h_all % world != 0:
      raise ValueError(f"heads ({h_all}) must be divisible by the context-parallel size ({world})")
    h_loc = h_all // world
    # peer j gets my sequence shard of its heads [j*h_loc, (j+1)*h_loc)
    send = x.reshape(b, world, h_loc, s_loc, d).permute(1, 0, 2, 3, 4).contiguous()
  else:
    h_loc, s_all = x.shape[1], x.shape[2]
    if s_all % world != 0:
      raise ValueError(f"sequence ({s_all}) must be divisible by the context-parallel size ({world})")
    s_loc = s_all // world
    # peer j gets its sequence shard of my heads
    send = x.reshape(b, h_loc, world, s_loc, d).permute(2, 0, 1, 3, 4).contiguous()
  recv = torch.empty_like(send)  # [P(source), B, h_loc, s_loc, D]
  dist.all_to_all_single(recv, send, group=group)
  if seq_to_head:  # source rank = sequence shard
    return recv.permute(1, 2, 0, 3, 4).reshape(b, h_loc, world * s_loc, d)
  return recv.permute(1, 0, 2, 3, 4).reshape(b, world * h_loc, s_loc, d)  # source rank = head block


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
  holds tokens ``[r*S/P, (r+1)*S/P)``.  ``P`` must divide the q-head count, and either divide the
  kv-head count too or be a multiple of it such that each rank's q heads read a single kv head (that
  head is then replicated); this keeps the reference's GQA mapping ``kv_head = q_head // (Hq / Hkv)``
  rank-local.  Returns the local sequence shard of the output ``[B, Hq, S/P, D]``.
  """

  def __init__(self, attention: Callable, group=None):
    self.attention = attention
    self.group = group

  @staticmethod
  def kv_heads_for_ranks(q_heads: int, kv_heads: int, world: int) -> list[int] | None:
    """None if ``world`` divides ``kv_heads`` (plain exchange); else the kv head each rank reads."""
    if q_heads % world != 0 or q_heads % kv_heads != 0:
      raise NotImplementedError(
          f"context-parallel size {world} must divide the q heads ({q_heads}), a multiple of the kv heads ({kv_heads})")
    if kv_heads % world == 0:
      return None
    per_rank, group = q_heads // world, q_heads // kv_heads
    if group % per_rank != 0:
      raise NotImplementedError(
          f"{world} ranks over {q_heads} q heads / {kv_heads} kv heads: a rank's q heads would read more than one kv "
          "head without owning any; use ring attention for this shape")
    return [(r * per_rank) // group for r in range(world)]

  def __call__(self, q, k, v, segment_ids: base.SegmentIds | None = None, *, logits_scale: float = 1.0):
    _, world = _world(self.group)
    replicate = self.kv_heads_for_ranks(q.shape[1], k.shape[1], world) if world > 1 else None
    if replicate is not None:
      index = torch.tensor(replicate, device=k.device)
      k, v = k.index_select(1, index), v.index_select(1, index)  # [B, P, S/P, D]: one head per destination
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
