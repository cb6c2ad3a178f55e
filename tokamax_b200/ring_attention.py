"""Ring attention: context parallelism with the keys and values sharded along the sequence.

Counterpart of the reference's ring wrapper
(tokamax/_src/ops/experimental/tpu/splash_attention/ring_attention_kernel.py:68-293, factory
:617-705).  Rank ``r`` of ``P`` keeps its query shard for the whole call and starts with key /
value shard ``r``; at step ``i`` it attends to shard ``(r - i) mod P`` and passes the shard it
holds on to rank ``r + 1`` (:98-113).  Per step the unsharded splash kernels run on the
(query shard, key shard) sub-mask; the forward merges the partial outputs through their
logsumexp in fp32 (:150-158), the backward calls the backward kernels with the merged output and
logsumexp, accumulates dq in place and sends the dk / dv accumulators round the ring with their
shard, so that they are back home after ``P`` steps (:228-262).

Unlike Ulysses (``tokamax_b200.ulysses``) this does not need ``P`` to divide the head counts and
never materialises the whole sequence on one GPU; it pays for that with ``P`` kernel launches per
pass and with merging in HBM.  The transfer of step ``i + 1``'s shard is posted before the kernels
of step ``i`` are launched, so it runs under them.

Differences from the reference: sub-masks are built per (query shard, key shard) pair from the
mask object itself (any mask, not only ``NumpyMask`` / ``FullMask``, :647-650), pairs whose
sub-mask is empty launch nothing, and tensors are batched ``[B, H, S / P, D]``.
"""

from __future__ import annotations

from typing import Any, Callable, Protocol

import numpy as np
import torch
import torch.distributed as dist

from tokamax_b200 import base
from tokamax_b200 import splash_attention_mask as mask_lib

DEFAULT_MASK_VALUE = base.DEFAULT_MASK_VALUE


# ----------------------------------------------------------------------------------------------
# sub-masks
# ----------------------------------------------------------------------------------------------
def shard_mask(mask: mask_lib.Mask, q_shard: int, kv_shard: int, q_shards: int, kv_shards: int) -> mask_lib.Mask:
  """The (q_shard, kv_shard) window of ``mask`` as a mask object of its own.

  Lazy masks stay lazy: a causal or local mask seen from a window is the same rule with its offset
  moved by ``q_start - kv_start``; a chunked-causal window is chunked-causal again on the diagonal
  when the shard length is a multiple of the chunk.  Anything else is materialised for the window.
  """
  q_len, kv_len = mask.shape
  if q_len % q_shards or kv_len % kv_shards:
    raise ValueError(f"mask {mask.shape} does not split into {q_shards} x {kv_shards} shards")
  sq, skv = q_len // q_shards, kv_len // kv_shards
  q0, k0 = q_shard * sq, kv_shard * skv
  shape = (sq, skv)
  if isinstance(mask, mask_lib.FullMask):
    return mask_lib.FullMask(shape)
  if isinstance(mask, mask_lib.CausalMask):
    return mask_lib.CausalMask(shape, offset=mask.offset + q0 - k0)
  if isinstance(mask, mask_lib.LocalMask):
    return mask_lib.LocalMask(shape, mask.window_size, mask.offset + q0 - k0)
  if isinstance(mask, mask_lib.ChunkedCausalMask) and q0 == k0 and q0 % mask.chunk_size == 0:
    return mask_lib.ChunkedCausalMask(shape, mask.chunk_size)
  if isinstance(mask, (mask_lib.LogicalAnd, mask_lib.LogicalOr)):
    return type(mask)(shard_mask(mask.left, q_shard, kv_shard, q_shards, kv_shards),
                      shard_mask(mask.right, q_shard, kv_shard, q_shards, kv_shards))
  window = np.ascontiguousarray(mask[q0:q0 + sq, k0:k0 + skv]).astype(np.bool_)
  return mask_lib.NumpyMask(window)


# ----------------------------------------------------------------------------------------------
# what the ring needs from the per-pair attention
# ----------------------------------------------------------------------------------------------
class ShardAttention(Protocol):
  """Attention of one query shard against one key shard."""

  empty: bool  # the sub-mask has no live block: both calls may be skipped

  def forward(self, q, k, v, q_seg, kv_seg, scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``(o [B, Hq, Sq, D], logsumexp fp32 [B, Hq, Sq])``; rows without a live key: lse <= -1e37."""

  def backward(self, q, k, v, o, lse, d_o, q_seg, kv_seg, scale: float):
    """``(dq, dk, dv)`` of this key shard given the merged ``o`` / ``lse``."""


class SplashShardAttention:
  """`ShardAttention` on the CUDA kernels."""

  def __init__(self, sub_mask: mask_lib.Mask, **kernel_kwargs):
    from tokamax_b200 import splash_attention_kernel as splash  # needs torch + the native library

    self._splash = splash
    self.kernel = splash.make_splash_mha(sub_mask, q_seq_shards=1, save_residuals=True, **kernel_kwargs)
    info = self.kernel.fwd_mask_info
    self.empty = info.num_active_blocks is not None and int(np.sum(info.num_active_blocks)) == 0
    if info.block_mask is not None and not self.empty:
      self.empty = not bool(np.any(np.asarray(info.block_mask) > 0))

  def forward(self, q, k, v, q_seg, kv_seg, scale):
    seg = None if q_seg is None else base.SegmentIds(q_seg, kv_seg)
    with torch.no_grad():
      o, res = self.kernel(q, k, v, seg, logits_scale=scale)
    return o, res["logsumexp"]

  def backward(self, q, k, v, o, lse, d_o, q_seg, kv_seg, scale):
    dq, dk, dv, _ = self._splash.splash_backward(self.kernel, q, k, v, o, lse, d_o, q_seg, kv_seg, scale)
    return dq, dk, dv


# ----------------------------------------------------------------------------------------------
# merge of partial softmaxes
# ----------------------------------------------------------------------------------------------
def merge_partial(o_acc: torch.Tensor, lse_acc: torch.Tensor, o_i: torch.Tensor, lse_i: torch.Tensor):
  """Folds one partial (normalised output, logsumexp) into the fp32 running pair, in place.

  Same arithmetic as the reference's (m, l, o) carry (:150-158) written on logsumexp: the merged
  output is the logsumexp-weighted mean of the partial outputs.
  """
  if o_acc.is_cuda:  # one fused pass (splash_ring_merge); the torch form below serves host tensors only
    if not (o_i.dtype == torch.bfloat16 and o_acc.shape[-1] == 128 and o_acc.is_contiguous()
            and o_i.is_contiguous() and lse_acc.is_contiguous() and lse_i.is_contiguous()):
      raise ValueError("merge_partial on a CUDA device takes contiguous fp32 / bf16 tensors with head_dim 128")
    import ctypes as C
    from tokamax_b200 import _native

    stream = C.c_void_p(torch.cuda.current_stream(o_acc.device).cuda_stream)
    with torch.cuda.device(o_acc.device):
      _native.check(_native.lib().splash_ring_merge(o_acc.data_ptr(), lse_acc.data_ptr(), o_i.data_ptr(),
                                                    lse_i.data_ptr(), lse_acc.numel(), 128, stream),
                    "splash_ring_merge")
    return
  # Weights from the larger of the two logsumexps, as in the kernel: exact also where both are the
  # (huge, finite) mask value, which `logaddexp` cannot move by log 2 in fp32.
  m = torch.maximum(lse_acc, lse_i)
  m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
  e_acc, e_i = torch.exp(lse_acc - m_safe), torch.exp(lse_i - m_safe)
  total = e_acc + e_i
  inv = torch.where(total > 0, 1.0 / total, torch.zeros_like(total))
  o_acc.mul_((e_acc * inv).unsqueeze(-1)).addcmul_(o_i.float(), (e_i * inv).unsqueeze(-1))
  lse_acc.copy_(torch.where(total > 0, m_safe + torch.log(total), m))


# ----------------------------------------------------------------------------------------------
# the ring
# ----------------------------------------------------------------------------------------------
def _ring_peers(group) -> tuple[int, int, int, int]:
  rank, world = dist.get_rank(group), dist.get_world_size(group)
  to_global = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
  return rank, world, to_global((rank + 1) % world), to_global((rank - 1) % world)


def _post_shift(tensors, group, nxt: int, prv: int):
  """Sends each tensor to the next rank and receives the previous rank's; returns (works, received)."""
  if nxt == prv == dist.get_rank():  # a ring of one: nothing moves
    return [], list(tensors)
  recv = [torch.empty_like(t) for t in tensors]
  ops = []
  for t, r in zip(tensors, recv):
    ops.append(dist.P2POp(dist.isend, t.contiguous(), nxt, group))
    ops.append(dist.P2POp(dist.irecv, r, prv, group))
  return dist.batch_isend_irecv(ops), recv


def _wait(works):
  for w in works:
    w.wait()


def _piece(t, idx: int, n: int, dim: int = 2):
  """Piece ``idx`` of ``n`` equal pieces of ``t`` along ``dim`` (``t`` itself when n == 1)."""
  if t is None or n == 1:
    return t
  size = t.shape[dim] // n
  return t.narrow(dim, idx * size, size)


def _seg_piece(t, idx: int, n: int):
  return None if t is None else _piece(t, idx, n, dim=1).contiguous()


class _RingFunction(torch.autograd.Function):
  """The ring over whole shards, each shard being one chunk (contiguous layout) or two (zig-zag)."""

  @staticmethod
  def forward(ctx, q, k, v, q_seg, kv_seg, ring, scale):
    rank, world, nxt, prv = _ring_peers(ring.group)
    b, hq, sq, d = q.shape
    q_chunks = ring.chunks_of(rank, world)
    nq = len(q_chunks)
    o_accs = [torch.zeros((b, hq, sq // nq, d), dtype=torch.float32, device=q.device) for _ in range(nq)]
    lse_accs = [torch.full((b, hq, sq // nq), -float("inf"), dtype=torch.float32, device=q.device) for _ in range(nq)]
    k_cur, v_cur, seg_cur = k.contiguous(), v.contiguous(), kv_seg
    for i in range(world):
      shard = (rank - i) % world
      works = None
      if i + 1 < world:  # the next step's shard travels under this step's kernels
        moving = [k_cur, v_cur] + ([seg_cur] if seg_cur is not None else [])
        works, received = _post_shift(moving, ring.group, nxt, prv)
      kv_chunks = ring.chunks_of(shard, world)
      nk = len(kv_chunks)
      for a, qc in enumerate(q_chunks):
        for c, kc in enumerate(kv_chunks):
          attn = ring.pair_attention(qc, kc, world)
          if attn.empty:
            continue
          o_i, lse_i = attn.forward(_piece(q, a, nq), _piece(k_cur, c, nk), _piece(v_cur, c, nk),
                                    _seg_piece(q_seg, a, nq), _seg_piece(seg_cur, c, nk), scale)
          merge_partial(o_accs[a], lse_accs[a], o_i, lse_i)
      if works is not None:
        _wait(works)
        k_cur, v_cur = received[0], received[1]
        seg_cur = received[2] if seg_cur is not None else None
    o_acc = o_accs[0] if nq == 1 else torch.cat(o_accs, dim=2)
    lse_acc = lse_accs[0] if nq == 1 else torch.cat(lse_accs, dim=2)
    dead = lse_acc < -1.0e37  # no live key on any shard (or no shard visited at all)
    o = torch.where(dead.unsqueeze(-1), torch.zeros_like(o_acc), o_acc).to(q.dtype)
    lse = torch.where(dead, torch.full_like(lse_acc, ring.mask_value), lse_acc)
    ctx.save_for_backward(q, k, v, o, lse, q_seg, kv_seg)
    ctx.ring, ctx.scale = ring, scale
    ctx.mark_non_differentiable(lse)
    return o, lse

  @staticmethod
  def backward(ctx, d_o, _dlse):
    q, k, v, o, lse, q_seg, kv_seg = ctx.saved_tensors
    ring, scale = ctx.ring, ctx.scale
    rank, world, nxt, prv = _ring_peers(ring.group)
    d_o = d_o.contiguous()
    q_chunks = ring.chunks_of(rank, world)
    nq = len(q_chunks)
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    lse_parts = [_piece(lse, a, nq).contiguous() for a in range(nq)]
    k_cur, v_cur, seg_cur = k.contiguous(), v.contiguous(), kv_seg
    acc_in_flight = None  # (works, [dk_acc, dv_acc]) on their way here from the previous rank
    for i in range(world):
      shard = (rank - i) % world
      works = None
      if i + 1 < world:
        moving = [k_cur, v_cur] + ([seg_cur] if seg_cur is not None else [])
        works, received = _post_shift(moving, ring.group, nxt, prv)
      kv_chunks = ring.chunks_of(shard, world)
      nk = len(kv_chunks)
      shares = []  # (kv piece, dk, dv) of this step
      for a, qc in enumerate(q_chunks):
        for c, kc in enumerate(kv_chunks):
          attn = ring.pair_attention(qc, kc, world)
          if attn.empty:
            continue
          dq_i, dk_i, dv_i = attn.backward(_piece(q, a, nq), _piece(k_cur, c, nk), _piece(v_cur, c, nk),
                                           _piece(o, a, nq), lse_parts[a], _piece(d_o, a, nq),
                                           _seg_piece(q_seg, a, nq), _seg_piece(seg_cur, c, nk), scale)
          _piece(dq, a, nq).add_(dq_i.float())
          shares.append((c, dk_i, dv_i))
      # The accumulators follow their shard: what the previous rank held for the shard now here
      # arrives while this step's kernels run, gets this step's share, and moves on.  After the
      # last step's shift they are home again (reference :255-262).
      if acc_in_flight is None:
        dk_acc = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
        dv_acc = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
      else:
        _wait(acc_in_flight[0])
        dk_acc, dv_acc = acc_in_flight[1]
      for c, dk_i, dv_i in shares:
        _piece(dk_acc, c, nk).add_(dk_i.float())
        _piece(dv_acc, c, nk).add_(dv_i.float())
      acc_in_flight = _post_shift([dk_acc, dv_acc], ring.group, nxt, prv)
      if works is not None:
        _wait(works)
        k_cur, v_cur = received[0], received[1]
        seg_cur = received[2] if seg_cur is not None else None
    _wait(acc_in_flight[0])
    dk_acc, dv_acc = acc_in_flight[1]
    return dq.to(q.dtype), dk_acc.to(k.dtype), dv_acc.to(v.dtype), None, None, None, None


class RingSplashAttention:
  """Sequence-sharded splash attention over a ring of ranks (reference :520-615).

  Call with the local shards ``q [B, Hq, S/P, D]``, ``k, v [B, Hkv, S/P, D]`` and optional
  ``SegmentIds`` shards ``[B, S/P]``.  Returns the local shard of the output, or
  ``(out, {"logsumexp"})`` with ``save_residuals=True``.

  ``layout="contiguous"`` (the reference's): rank ``r`` holds tokens ``[r S/P, (r+1) S/P)``.  Under
  a causal mask that ring is unbalanced — rank ``r`` has ``r + 1`` live (query, key) shard pairs.
  ``layout="zigzag"``: the sequence is cut into ``2P`` chunks and rank ``r`` holds chunks ``r`` and
  ``2P - 1 - r`` back to back (`zigzag_shard` / `zigzag_unshard` convert), which gives every rank
  the same number of live chunk pairs under a causal mask; results are the same attention.
  """

  def __init__(self, mask: mask_lib.Mask, *, group=None, save_residuals: bool = False,
               mask_value: float = DEFAULT_MASK_VALUE, layout: str = "contiguous",
               shard_attention_factory: Callable[[mask_lib.Mask], ShardAttention] | None = None,
               **kernel_kwargs: Any):
    if layout not in ("contiguous", "zigzag"):
      raise ValueError(f"layout must be 'contiguous' or 'zigzag', got {layout!r}")
    self.mask = mask
    self.layout = layout
    self.group = group
    self.save_residuals = save_residuals
    self.mask_value = max(float(mask_value), -3.0e38)
    self._factory = shard_attention_factory or (
        lambda sub: SplashShardAttention(sub, mask_value=mask_value, **kernel_kwargs))
    self._cache: dict[tuple[int, int, int], ShardAttention] = {}

  def chunks_of(self, rank: int, world: int) -> list[int]:
    """Sequence chunks (of ``n_chunks(world)``) held by ``rank``, in the order they are stored."""
    return [rank] if self.layout == "contiguous" else [rank, 2 * world - 1 - rank]

  def n_chunks(self, world: int) -> int:
    return world if self.layout == "contiguous" else 2 * world

  def pair_attention(self, q_chunk: int, kv_chunk: int, world: int) -> ShardAttention:
    n = self.n_chunks(world)
    key = (n, q_chunk, kv_chunk)
    if key not in self._cache:
      self._cache[key] = self._factory(shard_mask(self.mask, q_chunk, kv_chunk, n, n))
    return self._cache[key]

  def shard_attention(self, q_shard: int, kv_shard: int) -> ShardAttention:
    """Attention of (query shard, key shard) in the contiguous layout."""
    world = dist.get_world_size(self.group)
    key = (world, q_shard, kv_shard)
    if key not in self._cache:
      self._cache[key] = self._factory(shard_mask(self.mask, q_shard, kv_shard, world, world))
    return self._cache[key]

  def check_errors(self) -> None:
    """Raises if any of the per-pair kernels reported a device-side fault (see
    SplashAttentionKernel.check_errors)."""
    for attn in self._cache.values():
      kernel = getattr(attn, "kernel", None)
      if kernel is not None:
        kernel.check_errors()

  def __call__(self, q, k, v, segment_ids: base.SegmentIds | None = None, sinks=None, *,
               logits_scale: float = 1.0):
    if sinks is not None:
      raise NotImplementedError("Sinks aren't supported yet.")  # as the reference, :91-92
    world = dist.get_world_size(self.group)
    q_len, kv_len = self.mask.shape
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
      raise ValueError(f"expected [B, H, S/P, D] shards, got {tuple(q.shape)}, {tuple(k.shape)}")
    if q.shape[2] * world != q_len or k.shape[2] * world != kv_len or v.shape[2] != k.shape[2]:
      raise ValueError(f"shards of length {q.shape[2]} / {k.shape[2]} on {world} ranks do not tile the "
                       f"mask {self.mask.shape}")
    if q.shape[-1] != k.shape[-1]:
      raise NotImplementedError("Queries and keys must have the same head dimension.")
    q_seg = kv_seg = None
    if segment_ids is not None:
      q_seg = torch.as_tensor(segment_ids.q, device=q.device).to(torch.int32).contiguous()
      kv_seg = torch.as_tensor(segment_ids.kv, device=q.device).to(torch.int32).contiguous()
    out, lse = _RingFunction.apply(q, k, v, q_seg, kv_seg, self, float(logits_scale))
    if self.save_residuals:
      return out, {"logsumexp": lse}
    return out


def zigzag_shard(x: torch.Tensor, rank: int, world: int, dim: int = 2) -> torch.Tensor:
  """The zig-zag shard of rank ``rank``: chunks ``rank`` and ``2 world - 1 - rank`` of ``x`` along ``dim``."""
  chunks = x.chunk(2 * world, dim=dim)
  return torch.cat([chunks[rank], chunks[2 * world - 1 - rank]], dim=dim)


def zigzag_unshard(shards: list[torch.Tensor], dim: int = 2) -> torch.Tensor:
  """Inverse of `zigzag_shard` over the shards of all ranks, in rank order."""
  world = len(shards)
  chunks: list = [None] * (2 * world)
  for r, s in enumerate(shards):
    a, b = s.chunk(2, dim=dim)
    chunks[r], chunks[2 * world - 1 - r] = a, b
  return torch.cat(chunks, dim=dim)


def make_ring_attention(mask: np.ndarray | mask_lib.Mask, *, config=None, is_mqa: bool = False,
                        save_residuals: bool = False, mask_value: float = DEFAULT_MASK_VALUE,
                        downcast_smem_data: bool = True, partial_mask_blocks_dtype: Any = np.int8,
                        ring_axis=None, q_seq_shards: int = 1, kv_seq_shards: int = 1,
                        layout: str = "contiguous", repeatable_dq: bool = False) -> RingSplashAttention:
  """Reference factory (:617-705).  ``ring_axis`` is the process group of the ring (default: the
  world); ``layout`` is an addition (see `RingSplashAttention`)."""
  del q_seq_shards, kv_seq_shards  # the ring size is the group's size; sub-masks are cut per pair
  if len(mask.shape) != 2:
    raise ValueError(f"Unexpected mask shape: {mask.shape}")
  if isinstance(mask, np.ndarray):
    mask = mask_lib.NumpyMask(mask)
  if is_mqa:
    raise NotImplementedError("pass MQA keys / values with a kv-head axis of 1")
  kwargs = dict(downcast_smem_data=downcast_smem_data, partial_mask_blocks_dtype=partial_mask_blocks_dtype,
                repeatable_dq=repeatable_dq)
  if config is not None:
    kwargs["config"] = config
  return RingSplashAttention(mask, group=ring_axis, save_residuals=save_residuals, mask_value=mask_value,
                             layout=layout, **kwargs)
