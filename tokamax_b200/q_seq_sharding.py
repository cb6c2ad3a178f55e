"""Q-sequence sharding: one contiguous shard of the query rows per rank, keys and values replicated.

The reference builds per-shard MaskInfo tables with ``make_splash_mha(mask, q_seq_shards=n)`` and
runs shard ``i`` on device ``i`` under ``jax.shard_map`` with K / V unsharded along the sequence
(``splash_attention_kernel.py:2023-2053``, ``splash_attention_mask_info.py:494-544``; test
``splash_attention_kernel_sharded_test.py:60-150``).  Under shard_map the gradient of a replicated
input is summed over the mesh axis by the transpose of the replication; here that sum is an
all-reduce in the backward pass of K and V.  There is no exchange in the forward pass.

With a causal mask contiguous q shards are unbalanced (the last shard has the most live blocks);
``tokamax_b200.ulysses`` and ``tokamax_b200.ring_attention`` are the balanced schemes.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from tokamax_b200 import base


class _SumGradOverGroup(torch.autograd.Function):
  """Identity on a tensor every rank holds a copy of; its gradient is the sum of the ranks'."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return x.view_as(x)

  @staticmethod
  def backward(ctx, g):
    if dist.get_world_size(ctx.group) == 1:
      return g, None
    total = g.float().contiguous()  # each rank's share is a rounded bf16 tensor; add them in fp32
    dist.all_reduce(total, op=dist.ReduceOp.SUM, group=ctx.group)
    return total.to(g.dtype), None


class QSeqShardedSplashAttention:
  """Runs shard ``rank`` of a kernel built with ``q_seq_shards = world size``.

  Args:
    attention: a ``SplashAttentionKernel`` made with ``q_seq_shards=n``, or any callable
      ``(q, k, v, segment_ids, *, logits_scale, q_shard) -> out``.
    group: process group of the n ranks (default: the world).

  Call with this rank's rows ``q [B, Hq, S/n, D]`` (rank r holds rows ``[r*S/n, (r+1)*S/n)``), the
  whole ``k, v [B, Hkv, T, D]`` (the same on every rank) and, if any, ``SegmentIds(q=[B, S/n],
  kv=[B, T])``.  Returns this rank's rows of the output.  ``k.grad`` / ``v.grad`` come out summed
  over the ranks, i.e. complete and identical everywhere.
  """

  def __init__(self, attention: Callable, group=None):
    self.attention = attention
    self.group = group

  def __call__(self, q, k, v, segment_ids: base.SegmentIds | None = None, *, logits_scale: float = 1.0):
    rank, world = dist.get_rank(self.group), dist.get_world_size(self.group)
    shards = getattr(self.attention, "q_seq_shards", world)
    if shards != world:
      raise ValueError(f"the kernel was built for {shards} q shards, the group has {world} ranks")
    k = _SumGradOverGroup.apply(k, self.group)
    v = _SumGradOverGroup.apply(v, self.group)
    return self.attention(q, k, v, segment_ids, logits_scale=logits_scale, q_shard=rank)

  def check_errors(self) -> None:
    """Raises if the wrapped kernel reported a device-side fault (SplashAttentionKernel.check_errors)."""
    check = getattr(self.attention, "check_errors", None)
    if check is not None:
      check()
