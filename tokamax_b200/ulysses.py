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


class PeerExchange:
  """The same exchange by peer stores instead of a collective (``splash_exchange_push``).

  Receive buffers are symmetric-memory allocations (``torch.distributed._symmetric_memory``: every
  rank maps every other rank's buffer), laid out as the attention kernels read them; a rank copies
  its outgoing ``[S/P, D]`` slabs straight into its peers' buffers with its own copy kernel — plain
  16-byte loads and stores over NVLink, no TMA, no multicast — between two stream-ordered barriers
  (buffers free / all pushes landed; each a one-element NCCL all-reduce, so a rank that never
  arrives ends in NCCL's own timeout rather than in a spinning kernel).  Nothing is packed or
  unpacked.

  Buffers are cached per (tag, shape) and reused by the next call, so what a call leaves in them is
  only valid until the same tag is exchanged again: :class:`UlyssesSplashAttention` copies what it
  hands back to the caller (output, gradients) and gives each forward call whose backward is still
  pending its own set of buffers (``max_pending`` sets at most).
  """

  def __init__(self, group=None, max_pending: int = 4):
    import torch.distributed._symmetric_memory as symm_mem  # pylint: disable=g-import-not-at-top

    self._symm_mem = symm_mem
    self.group = group if group is not None else dist.group.WORLD
    self.max_pending = max_pending
    self._buffers: dict = {}
    self._pending: set[int] = set()
    self._flag: torch.Tensor | None = None

  def _barrier(self, device) -> None:
    if self._flag is None:
      self._flag = torch.zeros(1, dtype=torch.float32, device=device)
    dist.all_reduce(self._flag, group=self.group)  # enqueued on the current stream, ordered with the kernels around it

  def acquire(self, hold: bool) -> int:
    """A buffer-set index for one forward call; held until :meth:`release` if ``hold``."""
    slot = next(i for i in range(self.max_pending + 1) if i not in self._pending)
    if slot == self.max_pending:
      raise RuntimeError(f"{self.max_pending} forward calls are waiting for their backward; run backward (or call "
                         "under torch.no_grad()) before calling again, or raise max_pending")
    if hold:
      self._pending.add(slot)
    return slot

  def release(self, slot: int) -> None:
    self._pending.discard(slot)

  def _buffer(self, tag: str, shape, dtype, device):
    key = (tag, tuple(shape), dtype)
    if key not in self._buffers:
      t = self._symm_mem.empty(*shape, dtype=dtype, device=device)
      handle = self._symm_mem.rendezvous(t, self.group)  # collective: ranks create buffers in the same order
      # the mapped block may be larger than the tensor: where the tensor starts inside it
      base = t.data_ptr() - int(handle.buffer_ptrs[handle.rank])
      if base < 0 or base + t.numel() * t.element_size() > int(handle.buffer_size):
        raise RuntimeError(f"symmetric buffer for {tag}: tensor at {base} outside its block of {handle.buffer_size} bytes")
      self._buffers[key] = (t, handle, base)
    return self._buffers[key]

  def exchange(self, x: torch.Tensor, seq_to_head: bool, tag: str, barriers: tuple[bool, bool] = (True, True)) -> torch.Tensor:
    """``barriers``: whether this call runs the barrier before / after its copy kernel.  Exchanges
    issued back to back (q, k, v of one call) share one pair: the first keeps the barrier in front,
    the last the one behind, and nothing reads a received tensor before that last barrier."""
    import ctypes as C  # pylint: disable=g-import-not-at-top
    from tokamax_b200 import _native  # pylint: disable=g-import-not-at-top

    rank, world = _world(self.group)
    x = x.contiguous()
    b, d = x.shape[0], x.shape[3]
    if seq_to_head:
      if x.shape[1] % world:
        raise ValueError(f"heads ({x.shape[1]}) must be divisible by the context-parallel size ({world})")
      h_loc, s_loc = x.shape[1] // world, x.shape[2]
      out_shape = (b, h_loc, s_loc * world, d)
    else:
      if x.shape[2] % world:
        raise ValueError(f"sequence ({x.shape[2]}) must be divisible by the context-parallel size ({world})")
      h_loc, s_loc = x.shape[1], x.shape[2] // world
      out_shape = (b, h_loc * world, s_loc, d)
    out, handle, base = self._buffer(tag, out_shape, x.dtype, x.device)
    args = _native.SplashExchangeArgs()
    args.src, args.dst_ptrs = x.data_ptr(), int(handle.buffer_ptrs_dev)
    args.world, args.rank, args.seq_to_head = world, rank, int(seq_to_head)
    args.batch, args.h_loc, args.s_loc, args.row_bytes = b, h_loc, s_loc, d * x.element_size()
    args.dst_base_bytes = base
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
      if barriers[0]:
        self._barrier(x.device)  # every rank's earlier readers of its receive buffers are behind this point
      _native.check(_native.lib().splash_exchange_push(C.byref(args), C.c_void_p(stream)), "splash_exchange_push")
      if barriers[1]:
        self._barrier(x.device)  # every rank's stores have landed
    return out


def _run_exchange(x, group, seq_to_head: bool, engine, tag, barriers=(True, True)):
  if engine is None or dist.get_world_size(group) == 1:
    return _exchange(x, group, seq_to_head)
  return engine.exchange(x, seq_to_head, tag, barriers)


class _SeqToHead(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, group, engine=None, tag=None, barriers=(True, True)):
    ctx.group, ctx.engine, ctx.tag = group, engine, tag
    return _run_exchange(x, group, True, engine, tag, barriers)

  @staticmethod
  def backward(ctx, g):
    out = _run_exchange(g, ctx.group, False, ctx.engine, None if ctx.tag is None else ctx.tag + ".grad")
    if ctx.engine is not None:
      out = out.clone()  # handed to the caller as a .grad: must outlive the buffer's next use
    return out, None, None, None, None


class _HeadToSeq(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, group, engine=None, tag=None):
    ctx.group, ctx.engine, ctx.tag = group, engine, tag
    return _run_exchange(x, group, False, engine, tag)

  @staticmethod
  def backward(ctx, g):
    return _run_exchange(g, ctx.group, True, ctx.engine, None if ctx.tag is None else ctx.tag + ".grad"), None, None, None


def seq_to_head(x: torch.Tensor, group=None, engine: PeerExchange | None = None, tag: str | None = None,
                barriers: tuple[bool, bool] = (True, True)) -> torch.Tensor:
  """Differentiable all-to-all: sequence shard of all heads -> all of the sequence for H/P heads."""
  return _SeqToHead.apply(x, group, engine, tag, barriers)


def head_to_seq(x: torch.Tensor, group=None, engine: PeerExchange | None = None, tag: str | None = None) -> torch.Tensor:
  """Differentiable inverse of :func:`seq_to_head`."""
  return _HeadToSeq.apply(x, group, engine, tag)


def _peer_output(engine: "PeerExchange", tag: str, shape, like: torch.Tensor, head0: int):
  """(receive buffer of `shape` = [B, all heads, S/P, D], its SplashPeerOutput for this rank's head block)."""
  from tokamax_b200 import _native  # pylint: disable=g-import-not-at-top

  buf, handle, base = engine._buffer(tag, shape, like.dtype, like.device)  # pylint: disable=protected-access
  po = _native.SplashPeerOutput()
  po.ptrs, po.base_bytes, po.rows_per_peer = int(handle.buffer_ptrs_dev), base, shape[2]
  po.stride_b, po.stride_h, po.stride_s, po.head0 = buf.stride(0), buf.stride(1), buf.stride(2), head0
  return buf, po


class _FusedUlysses(torch.autograd.Function):
  """Sequence shards of q, k, v in, sequence shard of the output out, as one autograd node whose
  kernels write their results where they are needed.

  Forward: q, k, v reach the head layout by the copy kernel (three pushes, one pair of barriers); the
  forward kernel stores every output row into the local head-sharded `o` (the backward's residual)
  and, from its epilogue, into the receive buffer of the rank that owns the row
  (`SplashFwdArgs.o_peer`) — plain 16-byte stores over NVLink spread over the whole kernel — so the
  output's exchange costs one barrier.  Backward: dO comes in by the copy kernel; with the fused
  backward dK / dV rows leave from the epilogue of the kernel that accumulates them and dQ rows from
  the cast pass (`SplashBwdArgs.dq_peer / dk_peer / dv_peer`), again followed by one barrier; with
  the split backward (`repeatable_dq`) the three gradients are pushed (one pair of barriers).
  There is no device-side wait anywhere: ordering between ranks is the NCCL-ordered barriers.
  """

  @staticmethod
  def forward(ctx, q, k, v, owner, segment_ids, logits_scale):
    from tokamax_b200 import splash_attention_kernel as splash  # pylint: disable=g-import-not-at-top

    engine, kernel = owner.engine, owner.attention
    rank, world = _world(engine.group)
    needs_grad = any(ctx.needs_input_grad[:3])
    slot = engine.acquire(needs_grad)
    q_h = engine.exchange(q, True, f"q{slot}", (True, False))
    k_h = engine.exchange(k, True, f"k{slot}", (False, False))
    v_h = engine.exchange(v, True, f"v{slot}", (False, True))
    b, h_loc, s_all = q_h.shape[:3]
    s_loc = s_all // world
    out, po = _peer_output(engine, f"o{slot}", (b, h_loc * world, s_loc, v_h.shape[3]), q_h, rank * h_loc)
    stash = {}

    def into_peers(qh, kh, vh, q_seg, kv_seg, kern, scale, sinks, max_logit, shard):
      if sinks is not None or max_logit is not None or shard:
        raise NotImplementedError("sinks, a fixed maximum and q shards are not taken by the fused exchange")
      res = splash.splash_forward(kern, qh, kh, vh, q_seg, kv_seg, scale, None, None, 0, o_peer=po)
      stash.update(res=res[:5], seg=(q_seg, kv_seg), scale=scale)
      return out, res[4], res[5]

    # (the q / k / v pushes' barriers lie behind every rank's last read of its receive buffers)
    kernel(q_h, k_h, v_h, segment_ids, logits_scale=logits_scale, _function=into_peers)
    with torch.cuda.device(q.device):
      engine._barrier(q.device)  # every rank's forward has finished: all rows have landed  # pylint: disable=protected-access
    if needs_grad:
      qh, kh, vh, o_h, lse = stash["res"]
      q_seg, kv_seg = stash["seg"]
      ctx.save_for_backward(qh, kh, vh, o_h, lse, q_seg, kv_seg)
      ctx.kernel, ctx.scale, ctx.engine, ctx.slot = kernel, stash["scale"], engine, slot
      ctx.fuse_gradients = owner.fuse_gradients and not kernel.repeatable_dq
      ctx.shapes = (tuple(q.shape), tuple(k.shape), tuple(v.shape))
    return out.clone()  # the caller's tensor must outlive the buffer's next use

  @staticmethod
  def backward(ctx, g):
    from tokamax_b200 import splash_attention_kernel as splash  # pylint: disable=g-import-not-at-top

    q, k, v, o, lse, q_seg, kv_seg = ctx.saved_tensors
    engine, slot, kernel = ctx.engine, ctx.slot, ctx.kernel
    rank, _ = _world(engine.group)
    d_o = engine.exchange(g, True, f"o{slot}.grad")
    if not ctx.fuse_gradients:  # (the split backward's kernels have no second destination)
      dq_h, dk_h, dv_h, _ = splash.splash_backward(kernel, q, k, v, o, lse, d_o, q_seg, kv_seg, ctx.scale, 0)
      grads = [engine.exchange(dq_h, False, f"q{slot}.grad", (True, False)),
               engine.exchange(dk_h, False, f"k{slot}.grad", (False, False)),
               engine.exchange(dv_h, False, f"v{slot}.grad", (False, True))]
    else:
      outs = [_peer_output(engine, f"{name}{slot}.grad", shape, q, rank * heads)
              for name, shape, heads in zip("qkv", ctx.shapes, (q.shape[1], k.shape[1], v.shape[1]))]
      # (the dO push's barriers lie behind every rank's last read of these buffers)
      splash.splash_backward(kernel, q, k, v, o, lse, d_o, q_seg, kv_seg, ctx.scale, 0,
                             peers=tuple(po for _, po in outs))
      with torch.cuda.device(q.device):
        engine._barrier(q.device)  # every rank's backward has finished: all rows have landed  # pylint: disable=protected-access
      grads = [buf for buf, _ in outs]
    grads = [t.clone() for t in grads]  # handed to the caller as .grad: must outlive the buffers' next use
    engine.release(slot)
    return grads[0], grads[1], grads[2], None, None, None


class _ReleaseOnBackward(torch.autograd.Function):
  """Identity on q's path; its backward runs after the attention's, which is when the buffer set of
  the forward call is no longer needed."""

  @staticmethod
  def forward(ctx, x, engine, slot):
    ctx.engine, ctx.slot = engine, slot
    return x.view_as(x)

  @staticmethod
  def backward(ctx, g):
    ctx.engine.release(ctx.slot)
    return g, None, None


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
    exchange: "nccl" (default: one ``all_to_all_single`` per tensor), "peer" (:class:`PeerExchange`:
      own copy kernel over symmetric memory; CUDA + NVLink peers only) or "fused" ("peer", and the
      kernels themselves store the output, and with the fused backward the gradients, into the ranks
      that own the rows (:class:`_FusedUlysses`); needs a ``SplashAttentionKernel`` with head dims up
      to 128, falls back to "peer" otherwise).

  Call with the local sequence shards ``q [B, Hq, S/P, D]``, ``k, v [B, Hkv, S/P, D]``; rank ``r``
  holds tokens ``[r*S/P, (r+1)*S/P)``.  ``P`` must divide the q-head count, and either divide the
  kv-head count too or be a multiple of it such that each rank's q heads read a single kv head (that
  head is then replicated); this keeps the reference's GQA mapping ``kv_head = q_head // (Hq / Hkv)``
  rank-local.  Returns the local sequence shard of the output ``[B, Hq, S/P, D]``.
  """

  def __init__(self, attention: Callable, group=None, exchange: str = "nccl", fuse_gradients: bool = True):
    if exchange not in ("nccl", "peer", "fused"):
      raise ValueError(f"exchange must be 'nccl', 'peer' or 'fused', got {exchange!r}")
    self.attention = attention
    self.group = group
    self.engine = PeerExchange(group) if exchange in ("peer", "fused") else None
    self.fused = exchange == "fused"
    # "fused" only: whether dq / dk / dv also leave from the backward's kernels (else they are pushed)
    self.fuse_gradients = fuse_gradients

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
    engine = self.engine if world > 1 else None
    if engine is not None and self.fused and replicate is None and self._can_fuse(q, v):
      seg_full = None
      if segment_ids is not None:
        seg_full = base.SegmentIds(self._gather_seq(segment_ids.q), self._gather_seq(segment_ids.kv))
      return _FusedUlysses.apply(q, k, v, self, seg_full, logits_scale)
    tags = (None, None, None, None)
    if engine is not None:
      needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v))
      slot = engine.acquire(needs_grad)
      tags = tuple(f"{name}{slot}" for name in ("q", "k", "v", "o"))
      if needs_grad:
        q = _ReleaseOnBackward.apply(q, engine, slot)
    # the three pushes share one pair of barriers (nothing reads q_h / k_h / v_h before the last one)
    q_h = seq_to_head(q, self.group, engine, tags[0], (True, False))
    k_h = seq_to_head(k, self.group, engine, tags[1], (False, False))
    v_h = seq_to_head(v, self.group, engine, tags[2], (False, True))
    seg_full = None
    if segment_ids is not None:
      seg_full = base.SegmentIds(self._gather_seq(segment_ids.q), self._gather_seq(segment_ids.kv))
    o_h = self.attention(q_h, k_h, v_h, seg_full, logits_scale=logits_scale)
    out = head_to_seq(o_h, self.group, engine, tags[3])
    return out.clone() if engine is not None else out  # the caller's tensor must outlive the buffer's next use

  def _can_fuse(self, q_h, v_h) -> bool:
    from tokamax_b200 import splash_attention_kernel as splash  # pylint: disable=g-import-not-at-top

    a = self.attention
    return (isinstance(a, splash.SplashAttentionKernel) and q_h.shape[-1] <= 128 and v_h.shape[-1] <= 128 and
            q_h.dim() == 4 and not a.kwargs.get("save_residuals", False) and a.q_seq_shards == 1 and
            a.config.max_logit_const is None)

  def check_errors(self) -> None:
    """Raises if the wrapped kernel reported a device-side fault (SplashAttentionKernel.check_errors)."""
    check = getattr(self.attention, "check_errors", None)
    if check is not None:
      check()

  def _gather_seq(self, ids: torch.Tensor) -> torch.Tensor:
    _, world = _world(self.group)
    if world == 1:
      return ids
    ids = ids.contiguous()
    parts = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(parts, ids, group=self.group)
    return torch.cat(parts, dim=-1)
