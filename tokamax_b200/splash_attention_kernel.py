"""Splash attention on B200: the user-facing kernel objects.

Mirrors the public surface of the reference's
``tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_kernel.py``:
``QKVLayout`` (:103-111), ``SplashConfig`` (:114-196), ``SplashAttentionKernel`` (:2002-2067) and
the factories ``make_splash_mha`` / ``make_splash_mqa`` (+ ``_single_device``) (:2070-2131,
:2229-2237) and ``make_dynamic_splash_mha`` / ``_mqa`` (:2134-2226), with torch tensors in
place of ``jax.Array`` and ``torch.autograd`` in place of ``jax.custom_vjp`` (:998-1108,
:1871-1950).

All device work goes through the C ABI of ``libsplash_b200.so`` (``splash_fwd`` / ``splash_bwd``);
there is no PyTorch or CPU fallback — an unsupported configuration raises
``NotImplementedError`` and a missing CUDA device raises ``RuntimeError``.
"""

from __future__ import annotations

import ctypes as C
import dataclasses
import enum
import functools
from typing import Any

import numpy as np
import torch

from tokamax_b200 import _native
from tokamax_b200 import base
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import splash_attention_mask_info as mask_info_lib

SegmentIds = base.SegmentIds
MaskInfo = mask_info_lib.MaskInfo
DEFAULT_MASK_VALUE = base.DEFAULT_MASK_VALUE
partial = functools.partial

_TILE = 128
_HEAD_DIM = 128
_MAX_HEAD_DIM = 256  # above _HEAD_DIM: the kernels that work on two 128-column panels


def get_kernel_name(is_mqa: bool, save_residuals: bool, is_segmented: bool, phase: str) -> str:
  """Name of a kernel variant, in the reference's scheme (kernel.py:86-96)."""
  assert phase in ["dq", "dkv", "fwd"]
  assert not save_residuals or phase == "fwd"
  residuals = "_residuals" if save_residuals else "_no_residuals"
  attention_type = "mqa" if is_mqa else "mha"
  segments = "_segmented" if is_segmented else ""
  return f"splash_{attention_type}_{phase}{segments}{residuals}"


class QKVLayout(enum.IntEnum):
  HEAD_DIM_MINOR = enum.auto()  # [..., seq_len, head_dim]
  SEQ_MINOR = enum.auto()  # [..., head_dim, seq_len]


def from_head_minor(vals: tuple, layout: QKVLayout):
  """A shape (or any tuple) written head-dim-minor, as seen in ``layout``: the last two entries
  swap for SEQ_MINOR (reference kernel.py:108-111)."""
  if layout == QKVLayout.HEAD_DIM_MINOR:
    return vals
  return (*vals[:-2], vals[-1], vals[-2])


@dataclasses.dataclass(frozen=True, slots=True)
class SplashConfig:
  """Tile sizes and feature switches of the splash kernels (field-compatible with the reference).

  On B200 the MMA tile is fixed at 128x128; ``block_*`` choose the granularity of the MaskInfo
  tables (multiples of 128).  Fields that only steer the TPU code generator are accepted and
  ignored; fields that change results and are not built raise ``NotImplementedError`` at call
  time.
  """

  block_q: int
  block_kv: int
  block_kv_compute: int | None = None

  block_q_dkv: int | None = None
  block_kv_dkv: int | None = None
  block_kv_dkv_compute: int | None = None

  block_q_dq: int | None = None
  block_kv_dq: int | None = None
  use_fused_bwd_kernel: bool = True
  num_stacked_q_heads: int = 1
  q_layout: QKVLayout = QKVLayout.HEAD_DIM_MINOR
  k_layout: QKVLayout = QKVLayout.HEAD_DIM_MINOR
  v_layout: QKVLayout = QKVLayout.HEAD_DIM_MINOR

  fwd_cost_estimate: Any = None
  bwd_cost_estimate: Any = None

  residual_checkpoint_name: str | None = None
  attn_logits_soft_cap: float | None = None
  fuse_reciprocal: bool = True
  use_base2_exp: bool = True
  max_logit_const: float | None = None
  interpret: bool = False
  dq_reduction_steps: int | None = None
  use_experimental_scheduler: bool = False

  def __post_init__(self):
    if self.block_kv_compute is None:
      object.__setattr__(self, "block_kv_compute", self.block_kv)
    if self.block_kv_dkv_compute is None:
      object.__setattr__(self, "block_kv_dkv_compute", self.block_kv_dkv)
    if self.dq_reduction_steps is not None and self.dq_reduction_steps != 3:
      raise ValueError(
          f"Invalid dq_reduction_steps: {self.dq_reduction_steps}, only 3 or None are supported."
      )
    if not self.use_fused_bwd_kernel:
      raise ValueError("Only the fused bwd kernel is supported.")

  @property
  def has_backward_blocks(self) -> bool:
    return all(b is not None for b in (self.block_q_dkv, self.block_kv_dkv, self.block_kv_dkv_compute))

  @classmethod
  def get_default(cls):
    return SplashConfig(
        block_q=128, block_kv=128, block_kv_compute=128,
        block_q_dkv=128, block_kv_dkv=128, block_kv_dkv_compute=128,
        block_q_dq=128, block_kv_dq=128, fuse_reciprocal=True,
    )


# ----------------------------------------------------------------------------------------------
# device-side tables
# ----------------------------------------------------------------------------------------------
def _require_cuda(t: torch.Tensor) -> None:
  if not t.is_cuda:
    raise RuntimeError(
        "splash attention runs on CUDA (sm_100a) only and has no CPU path; got a tensor on "
        f"{t.device}"
    )


def _build_schedule(state: np.ndarray, pid: np.ndarray, block_q: int, block_kv: int, kind: int):
  out = _native.SplashScheduleOut()
  lib = _native.lib()
  state = np.ascontiguousarray(state, dtype=np.int32)
  pid = np.ascontiguousarray(pid, dtype=np.int32)
  _native.check(
      lib.splash_schedule_build(state.ctypes.data, pid.ctypes.data, state.shape[0], state.shape[1],
                                block_q, block_kv, kind, C.byref(out)),
      "splash_schedule_build",
  )
  try:
    row_ptr = np.ctypeslib.as_array(out.row_ptr, shape=(out.n_rows + 1,)).copy()
    n = max(int(out.n_entries), 1)
    entries = np.ctypeslib.as_array(out.entries, shape=(n * 4,)).copy()
    if out.n_entries == 0:
      entries[:] = 0
    row_order = np.ctypeslib.as_array(out.row_order, shape=(out.n_rows,)).copy()
  finally:
    lib.splash_schedule_free(C.byref(out))
  return row_ptr, entries, row_order


class _DeviceTables:
  """Schedules, partial-mask blocks and the error record of one kernel object on one device."""

  def __init__(self, kernel: "SplashAttentionKernel", device: torch.device, shard: int = 0):
    cfg = kernel.config
    fwd, dkv = kernel.fwd_mask_info, kernel.dkv_mask_info
    n_shards = kernel.q_seq_shards
    q_len, kv_len = kernel.mask_shape
    q_len //= n_shards  # the q rows of this shard; keys are never sharded here
    for b in (cfg.block_q, cfg.block_kv):
      if b % _TILE != 0:
        raise NotImplementedError(f"block sizes must be multiples of {_TILE} on B200, got {b}")
    nq, nkv = q_len // cfg.block_q, kv_len // cfg.block_kv
    state, pid = mask_info_lib.block_grids(fwd, nq, nkv, is_dkv=False, shard=shard, n_shards=n_shards)
    self.keep = []
    self.fwd = self._upload(state, pid, cfg.block_q, cfg.block_kv, 0, fwd.partial_mask_blocks, device)
    self.dq = self._upload(state, pid, cfg.block_q, cfg.block_kv, 1, fwd.partial_mask_blocks, device)
    if dkv is not None:
      bq, bkv = cfg.block_q_dkv, cfg.block_kv_dkv
      for b in (bq, bkv):
        if b % _TILE != 0:
          raise NotImplementedError(f"block sizes must be multiples of {_TILE} on B200, got {b}")
      st2, pid2 = mask_info_lib.block_grids(dkv, q_len // bq, kv_len // bkv, is_dkv=True, shard=shard, n_shards=n_shards)
      self.dkv = self._upload(st2, pid2, bq, bkv, 2, dkv.partial_mask_blocks, device)
    else:
      pmb_t = None
      if fwd.partial_mask_blocks is not None:
        pmb_t = np.ascontiguousarray(np.swapaxes(np.asarray(fwd.partial_mask_blocks), -1, -2))
      self.dkv = self._upload(state, pid, cfg.block_q, cfg.block_kv, 2, pmb_t, device)
    self.error_record = torch.zeros(4, dtype=torch.int32, device=device)
    q_seq = fwd.q_sequence
    if q_seq is not None and n_shards > 1:  # global q indices of this shard's rows
      q_seq = np.asarray(q_seq)[shard * q_len:(shard + 1) * q_len]
    self.q_sequence = None
    if q_seq is not None and not np.array_equal(np.asarray(q_seq), np.arange(q_len, dtype=np.int32)):
      self.q_sequence = torch.from_numpy(np.ascontiguousarray(q_seq, dtype=np.int32)).to(device)

  def _upload(self, state, pid, bq, bkv, kind, pmb, device) -> _native.SplashDeviceSchedule:
    row_ptr, entries, row_order = _build_schedule(state, pid, bq, bkv, kind)
    rp = torch.from_numpy(row_ptr).to(device)
    en = torch.from_numpy(entries).to(device)
    ro = torch.from_numpy(row_order).to(device)
    self.keep += [rp, en, ro]
    d = _native.SplashDeviceSchedule()
    d.row_ptr = rp.data_ptr()
    d.entries = en.data_ptr()
    d.row_order = ro.data_ptr()
    d.n_rows = len(row_ptr) - 1
    d.n_entries = int(row_ptr[-1])
    d.block_q, d.block_kv = bq, bkv
    d.partial_mask_blocks = None
    if pmb is not None:
      pm = torch.from_numpy(np.ascontiguousarray(np.asarray(pmb), dtype=np.int8)).to(device)
      self.keep.append(pm)
      d.partial_mask_blocks = pm.data_ptr()
    return d


class _DynamicDeviceTables:
  """Schedules built on the device from a mask tensor (no host round trip; one per batch size).

  The 128x128 tile states come from one pass over the mask, the three schedules from one small
  kernel each, and partial tiles are read from the mask itself (its transpose for dkv).
  """

  def __init__(self, mask: torch.Tensor, batch: int):
    lib = _native.lib()
    device = mask.device
    if mask.dim() != 2 or mask.dtype not in (torch.bool, torch.int8, torch.uint8):
      raise ValueError(f"expected a 2-dim bool / int8 mask tensor, got {mask.dtype} {tuple(mask.shape)}")
    q_len, kv_len = mask.shape
    if q_len % _TILE or kv_len % _TILE:
      raise NotImplementedError(f"mask sides must be multiples of {_TILE} on B200, got {tuple(mask.shape)}")
    # Snapshot: the kernels read the mask in place on every call, so a copy is kept; a caller who
    # updates its tensor afterwards builds a new kernel object.
    m = mask.contiguous().view(torch.uint8).clone()
    mt = m.t().contiguous()
    if mt.data_ptr() % 16:
      mt = mt.clone()
    states = torch.empty((q_len // _TILE, kv_len // _TILE), dtype=torch.int32, device=device)
    stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    self.keep = [m, mt, states]
    with torch.cuda.device(device):
      _native.check(lib.splash_mask_tile_states(m.data_ptr(), m.stride(0), q_len, kv_len, states.data_ptr(), stream),
                    "splash_mask_tile_states")
      scheds = []
      for kind, blocks in ((0, m), (1, m), (2, mt)):
        nbytes = lib.splash_dynamic_schedule_bytes(q_len, kv_len, kind, batch)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        out = _native.SplashDeviceSchedule()
        _native.check(lib.splash_dynamic_schedule(states.data_ptr(), q_len, kv_len, kind, batch, blocks.data_ptr(),
                                                  ws.data_ptr(), nbytes, C.byref(out), stream),
                      "splash_dynamic_schedule")
        self.keep.append(ws)
        scheds.append(out)
    self.fwd, self.dq, self.dkv = scheds
    self.tile_states = states
    self.error_record = torch.zeros(4, dtype=torch.int32, device=device)
    self.q_sequence = None


def _segment_schedule(sched: _native.SplashDeviceSchedule, kind: int, q_seg, kv_seg, q_len: int, kv_len: int):
  """Per-batch-row copy of ``sched`` without the tiles the segment ids rule out (device side).

  Returns ``(schedule, workspace tensor to keep alive)``; with no entries at all the input
  schedule is returned unchanged.
  """
  if sched.n_entries == 0:
    return sched, None
  lib = _native.lib()
  batch = q_seg.shape[0]
  nbytes = lib.splash_segment_schedule_bytes(batch, q_len, kv_len, sched.n_rows, sched.n_entries)
  ws = torch.empty(nbytes, dtype=torch.uint8, device=q_seg.device)
  out = _native.SplashDeviceSchedule()
  stream = torch.cuda.current_stream(q_seg.device).cuda_stream
  with torch.cuda.device(q_seg.device):
    _native.check(
        lib.splash_segment_schedule(C.byref(sched), kind, q_seg.data_ptr(), kv_seg.data_ptr(), batch, q_len, kv_len,
                                    ws.data_ptr(), nbytes, C.byref(out), C.c_void_p(stream)),
        "splash_segment_schedule")
  return out, ws


def _tensor_desc(t: torch.Tensor) -> _native.SplashTensor:
  d = _native.SplashTensor()
  d.data = t.data_ptr()
  d.dtype = 0
  for i in range(4):
    d.size[i] = t.shape[i]
    d.stride[i] = t.stride(i)
  return d


def _usable(t: torch.Tensor) -> torch.Tensor:
  """Returns ``t`` if the kernels can read it in place, else a contiguous copy."""
  ok = t.stride(-1) == 1 and all(s % 8 == 0 for s in t.stride()[:-1]) and t.data_ptr() % 16 == 0
  return t if ok else t.contiguous()


def _mask_fn_struct(mask_function_rule) -> _native.SplashMaskFn:
  fn = _native.SplashMaskFn()
  if mask_function_rule is not None:
    for name, value in zip(mask_function_rule._fields, mask_function_rule):
      setattr(fn, name, int(value))
  return fn


def splash_forward(kernel, q, k, v, q_seg, kv_seg, scale, sinks, max_logit, shard=0, o_peer=None):
  """One `splash_fwd` call on batched ``[B, H, S, D]`` bf16 tensors.

  Returns ``(q, k, v, o, logsumexp, max_logits, sinks_f32)``: the operands as the kernel read them
  (copies where a tensor could not be read in place) and the results.  ``o_peer``: an optional
  `_native.SplashPeerOutput`, the second destination of ``o`` in other ranks' memory.
  """
  _require_cuda(q)
  tables = kernel._tables(q.device, q.shape[0], shard)  # pylint: disable=protected-access
  q, k, v = _usable(q), _usable(k), _usable(v)
  b, hq, sq, d = q.shape
  if v.shape[-1] == d:
    o = torch.empty_like(q)  # keeps q's (dense) stride order, e.g. [B,T,H,D] storage stays [B,T,H,D]
  else:
    o = torch.empty((b, hq, sq, v.shape[-1]), dtype=q.dtype, device=q.device)
  lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
  max_logits = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
  args = _native.SplashFwdArgs()
  args.q, args.k, args.v, args.o = map(_tensor_desc, (q, k, v, o))
  args.logsumexp = lse.data_ptr()
  args.max_logits = max_logits.data_ptr()
  args.q_segment_ids = q_seg.data_ptr() if q_seg is not None else None
  args.kv_segment_ids = kv_seg.data_ptr() if kv_seg is not None else None
  args.q_sequence = tables.q_sequence.data_ptr() if tables.q_sequence is not None else None
  keep = []
  args.sched = tables.fwd
  if q_seg is not None and not tables.fwd.row_end:  # device-built schedules are not filtered further
    args.sched, ws = _segment_schedule(tables.fwd, 0, q_seg, kv_seg, q.shape[2], k.shape[2])
    keep.append(ws)
  args.mask_fn = _mask_fn_struct(kernel.mask_function_rule)
  args.scale = scale
  args.mask_value = max(kernel.mask_value, -3.0e38)
  args.error_record = tables.error_record.data_ptr()
  sinks_f32 = None if sinks is None else sinks.detach().to(torch.float32).contiguous()
  args.sinks = None if sinks_f32 is None else sinks_f32.data_ptr()
  args.soft_cap = float(kernel.config.attn_logits_soft_cap or 0.0)
  args.max_logit_value = None if max_logit is None else max_logit.data_ptr()
  if o_peer is not None:
    args.o_peer = o_peer
  stream = torch.cuda.current_stream(q.device).cuda_stream
  with torch.cuda.device(q.device):
    _native.check(_native.lib().splash_fwd(C.byref(args), C.c_void_p(stream)), "splash_fwd")
  return q, k, v, o, lse, max_logits, sinks_f32


class _SplashFunction(torch.autograd.Function):
  """forward = splash_fwd, backward = splash_bwd (reference custom_vjp: kernel.py:998-1108)."""

  @staticmethod
  def forward(ctx, q, k, v, q_seg, kv_seg, kernel, scale, sinks, max_logit, shard=0):
    q, k, v, o, lse, max_logits, sinks_f32 = splash_forward(kernel, q, k, v, q_seg, kv_seg, scale, sinks, max_logit, shard)
    ctx.save_for_backward(q, k, v, o, lse, q_seg, kv_seg, sinks_f32)
    ctx.sinks_dtype = None if sinks is None else sinks.dtype
    ctx.kernel = kernel
    ctx.scale = scale
    ctx.shard = shard
    ctx.mark_non_differentiable(lse, max_logits)
    return o, lse, max_logits

  @staticmethod
  def backward(ctx, d_o, _dlse, _dmax):
    q, k, v, o, lse, q_seg, kv_seg, sinks = ctx.saved_tensors
    dq, dk, dv, neg_di = splash_backward(ctx.kernel, q, k, v, o, lse, d_o, q_seg, kv_seg, ctx.scale, ctx.shard)
    dsinks = None
    if sinks is not None:
      # reference kernel.py:1928-1935: dsinks[h] = -sum_rows exp(sink - lse) * sum_d(o * do)
      dsinks = (torch.exp(sinks[None, :, None] - lse) * neg_di).sum(dim=(0, 2)).to(ctx.sinks_dtype)
    return dq, dk, dv, None, None, None, None, dsinks, None, None


def splash_backward(kernel: "SplashAttentionKernel", q, k, v, o, lse, d_o, q_seg=None, kv_seg=None,
                    scale: float = 1.0, shard: int = 0, peers=None):
  """One `splash_bwd` call: ``(dq, dk, dv, neg_di)`` for batched ``[B, H, S, 128]`` bf16 tensors.

  ``peers``: optional ``(dq_peer, dk_peer, dv_peer)`` of `_native.SplashPeerOutput`, second
  destinations of the gradients in other ranks' memory (fused backward only).

  ``o`` and ``lse`` are the forward's output and logsumexp for these q rows; they may come from a
  softmax over more keys than ``k`` holds (ring attention passes the merged values, reference
  ring_attention_kernel.py:228-262), in which case dq / dk / dv are this key shard's share.
  ``neg_di`` is ``-sum_d(o * do)`` (fp32 ``[B, Hq, Sq]``), a view of the backward's workspace, which
  keeps the row sums negated.
  """
  tables = kernel._tables(q.device, q.shape[0], shard)  # pylint: disable=protected-access
  d_o = _usable(d_o)
  dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
  lib = _native.lib()
  # head dims above 128 run three separate passes (dq, dk, dv), each repeatable bit for bit
  fused = not kernel.repeatable_dq and q.shape[-1] <= _HEAD_DIM and v.shape[-1] <= _HEAD_DIM
  size_fn = lib.splash_bwd_fused_workspace_bytes if fused else lib.splash_bwd_workspace_bytes
  ws_bytes = size_fn(q.shape[0], q.shape[1], q.shape[2])
  workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
  args = _native.SplashBwdArgs()
  args.flags = _native.BWD_FUSED_DQ if fused else 0
  args.q, args.k, args.v, args.o, args.d_o = map(_tensor_desc, (q, k, v, o, d_o))
  args.dq, args.dk, args.dv = map(_tensor_desc, (dq, dk, dv))
  args.logsumexp = lse.data_ptr()
  args.q_segment_ids = q_seg.data_ptr() if q_seg is not None else None
  args.kv_segment_ids = kv_seg.data_ptr() if kv_seg is not None else None
  args.q_sequence = tables.q_sequence.data_ptr() if tables.q_sequence is not None else None
  keep = []
  args.sched_dq = tables.dq
  args.sched_dkv = tables.dkv
  if q_seg is not None and not tables.dq.row_end:
    if not fused:  # the fused form walks the dkv schedule only
      args.sched_dq, ws1 = _segment_schedule(tables.dq, 1, q_seg, kv_seg, q.shape[2], k.shape[2])
      keep.append(ws1)
    args.sched_dkv, ws2 = _segment_schedule(tables.dkv, 2, q_seg, kv_seg, q.shape[2], k.shape[2])
    keep.append(ws2)
  args.mask_fn = _mask_fn_struct(kernel.mask_function_rule)
  args.scale = scale
  args.workspace = workspace.data_ptr()
  args.workspace_bytes = ws_bytes
  args.soft_cap = float(kernel.config.attn_logits_soft_cap or 0.0)
  args.error_record = tables.error_record.data_ptr()
  if peers is not None:
    args.dq_peer, args.dk_peer, args.dv_peer = peers
  stream = torch.cuda.current_stream(q.device).cuda_stream
  with torch.cuda.device(q.device):
    _native.check(lib.splash_bwd(C.byref(args), C.c_void_p(stream)), "splash_bwd")
  n = q.shape[0] * q.shape[1] * q.shape[2]
  neg_di = workspace[:4 * n].view(torch.float32).view(q.shape[0], q.shape[1], q.shape[2])
  return dq, dk, dv, neg_di


class SplashAttentionKernel:
  """Callable splash attention for one mask (reference: kernel.py:2002-2067).

  ``kernel(q, k, v, segment_ids=None, sinks=None, *, max_logit_value=None, logits_scale=1.0)``
  with q ``[q_heads, q_len, 128]`` (or batched ``[batch, q_heads, q_len, 128]``), k / v
  ``[kv_heads, kv_len, 128]`` (``[kv_len, 128]`` for MQA), bf16 on a CUDA device.  Returns ``out``,
  or ``(out, {"logsumexp", "max_logits"})`` when built with ``save_residuals=True``.  As in the
  reference no softmax scale is applied unless ``logits_scale`` is given (an extension that folds
  the caller's ``q * scale`` into the kernel in fp32).  Differentiable through torch autograd.
  """

  def __init__(self, fwd_mask_info: MaskInfo | None, dkv_mask_info: MaskInfo | None, *,
               dynamic_mask: torch.Tensor | None = None, **kwargs):
    self.kwargs = kwargs
    self._fwd_mask_info = fwd_mask_info
    self._dkv_mask_info = dkv_mask_info
    # A mask tensor on a CUDA device: schedules are built there at call time, and the MaskInfo
    # tables (host arrays, for inspection / pytree parity) only if somebody asks for them.
    self._dynamic_mask = dynamic_mask
    self._device_tables: dict = {}

  def _dynamic_info(self, is_dkv: bool) -> MaskInfo:
    cfg = self.config
    block = (cfg.block_q_dkv, cfg.block_kv_dkv) if is_dkv else (cfg.block_q, cfg.block_kv)
    return mask_info_lib._process_dynamic_mask(self._dynamic_mask, block, is_dkv=is_dkv)  # pylint: disable=protected-access

  @property
  def fwd_mask_info(self) -> MaskInfo:
    if self._fwd_mask_info is None and self._dynamic_mask is not None:
      self._fwd_mask_info = self._dynamic_info(False)
    return self._fwd_mask_info

  @property
  def dkv_mask_info(self) -> MaskInfo | None:
    if self._dkv_mask_info is None and self._dynamic_mask is not None and self.config.has_backward_blocks:
      self._dkv_mask_info = self._dynamic_info(True)
    return self._dkv_mask_info

  # attribute views of kwargs
  config = property(lambda self: self.kwargs["config"])
  is_mqa = property(lambda self: self.kwargs["is_mqa"])
  save_residuals = property(lambda self: self.kwargs.get("save_residuals", False))
  mask_value = property(lambda self: self.kwargs.get("mask_value", DEFAULT_MASK_VALUE))
  mask_function = property(lambda self: self.kwargs.get("mask_function"))
  mask_function_rule = property(lambda self: self.kwargs.get("mask_function_rule"))
  mask_shape = property(lambda self: self.kwargs["mask_shape"])
  # False (default): the fused backward — one kernel, five matmuls per live block like the
  # reference's (kernel.py:1234-1459), dq partials summed by fp32 reductions whose order varies
  # between runs.  True: separate dq and dkv kernels, every gradient bitwise repeatable.
  repeatable_dq = property(lambda self: bool(self.kwargs.get("repeatable_dq", False)))
  # > 1: the MaskInfo tables hold one segment per contiguous q-sequence shard (reference
  # kernel.py:2023-2053 hands shard i of them to device i under shard_map); a call then takes the
  # q rows of ONE shard ([.., q_len / shards, 128], `q_shard=i`) against all keys.
  q_seq_shards = property(lambda self: int(self.kwargs.get("q_seq_shards", 1)))

  def with_options(self, **kwargs) -> "SplashAttentionKernel":
    """A kernel object for the same mask with some keyword options replaced (``repeatable_dq``,
    ``save_residuals``, ``mask_value``); device tables and the error record are shared."""
    other = SplashAttentionKernel(self._fwd_mask_info, self._dkv_mask_info, dynamic_mask=self._dynamic_mask,
                                  **dict(self.kwargs, **kwargs))
    other._device_tables = self._device_tables  # pylint: disable=protected-access
    return other

  def _tables(self, device: torch.device, batch: int = 1, shard: int = 0):
    if shard and (self._dynamic_mask is not None or not 0 <= shard < self.q_seq_shards):
      raise ValueError(f"q shard {shard} does not exist in a kernel built with q_seq_shards={self.q_seq_shards}")
    if self._dynamic_mask is not None:
      if self._dynamic_mask.device != device:
        raise ValueError(f"the mask lives on {self._dynamic_mask.device}, the inputs on {device}")
      key = (device.type, device.index, int(batch))
      if key not in self._device_tables:
        self._device_tables[key] = _DynamicDeviceTables(self._dynamic_mask, int(batch))
      return self._device_tables[key]
    key = (device.type, device.index, shard) if self.q_seq_shards > 1 else (device.type, device.index)
    if key not in self._device_tables:
      self._device_tables[key] = _DeviceTables(self, device, shard)
    return self._device_tables[key]

  def check_errors(self) -> None:
    """Synchronises and raises if a kernel reported a device-side fault (bounded wait ran out).

    While a record holds an error, every kernel launched with it returns at once and leaves its
    outputs unwritten, so results produced since the fault are garbage.  Raising clears the
    record: the kernel object is usable again afterwards.
    """
    lib = _native.lib()
    for tables in self._device_tables.values():
      rec = (C.c_uint32 * 4)()
      dev = tables.error_record.device
      stream = torch.cuda.current_stream(dev).cuda_stream
      with torch.cuda.device(dev):
        st = lib.splash_read_error(tables.error_record.data_ptr(), C.c_void_p(stream), C.byref(rec))
      if st != 0:
        tables.error_record.zero_()
        raise _native.SplashError(st, f"device error record {list(rec)}")

  def _reject_unsupported(self, q, k, sinks, max_logit_value):
    cfg = self.config
    if cfg.max_logit_const is not None and max_logit_value is not None:
      raise ValueError(f"Only one of max_logit_const={cfg.max_logit_const} and {max_logit_value=} can be set.")
    if cfg.attn_logits_soft_cap is not None and not cfg.attn_logits_soft_cap > 0:
      raise ValueError(f"attn_logits_soft_cap must be positive, got {cfg.attn_logits_soft_cap}")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16:
      raise NotImplementedError(f"only bfloat16 inputs are built on B200, got {q.dtype}")

  def __call__(self, q, k, v, segment_ids: SegmentIds | None = None, sinks=None, *,
               max_logit_value=None, logits_scale: float = 1.0, q_shard: int = 0, _function=None, **overrides):
    # `_function`: what runs on the checked arguments in place of the plain autograd function (the
    # context-parallel wrapper passes one whose forward also stores the output into its peers).
    kw = dict(self.kwargs, **overrides)
    save_residuals = kw.get("save_residuals", False)
    self._reject_unsupported(q, k, sinks, max_logit_value)
    # SEQ_MINOR operands ([..., head_dim, seq], reference kernel.py:51-54) are viewed head-dim-minor;
    # the kernels take head_dim-contiguous tiles, so such an operand is copied once on the way in.
    cfg = self.config
    if cfg.q_layout == QKVLayout.SEQ_MINOR:
      q = q.transpose(-1, -2)
    if cfg.k_layout == QKVLayout.SEQ_MINOR:
      k = k.transpose(-1, -2)
    if cfg.v_layout == QKVLayout.SEQ_MINOR:
      v = v.transpose(-1, -2)
    batched = q.dim() == 4
    is_mqa = self.is_mqa
    if not batched:
      q = q[None]
      k, v = k[None], v[None]
    if is_mqa:
      if k.dim() != 3:
        raise ValueError(f"MQA expects k/v without a head axis, got k of rank {k.dim() - 1}")
      k, v = k[:, None], v[:, None]
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
      raise ValueError(f"Unexpected ranks: q {q.shape}, k {k.shape}, v {v.shape}")
    q_len, kv_len = self.mask_shape
    q_len //= self.q_seq_shards
    if q.shape[2] != q_len or k.shape[2] != kv_len or v.shape[2] != kv_len:
      raise ValueError(f"Sequence lengths {q.shape[2]}, {k.shape[2]} do not match the mask {self.mask_shape}"
                       + (f" cut into {self.q_seq_shards} q shards" if self.q_seq_shards > 1 else ""))
    if k.shape[1] == 0 or q.shape[1] % k.shape[1] != 0:
      raise ValueError(f"q heads ({q.shape[1]}) must be a multiple of kv heads ({k.shape[1]})")
    # The MMA tiles are 128 wide.  Smaller head dims (multiples of 8; q / k and v may differ) are
    # read in place: the kernels' TMA boxes reach past the end of a row and get zeros there, which
    # change neither q k^T nor p v, and only the real columns of outputs and gradients are stored.
    # No copy is made.  Head dims above 128, up to 256 (the reference's (192, 128) and (256, 256)),
    # run kernels that work on two 128-column panels.
    d_qk, d_v = q.shape[-1], v.shape[-1]
    if k.shape[-1] != d_qk:
      raise ValueError(f"q and k head dims differ: {d_qk} vs {k.shape[-1]}")
    if d_qk > _MAX_HEAD_DIM or d_v > _MAX_HEAD_DIM:
      raise NotImplementedError(f"head dims above {_MAX_HEAD_DIM} are not built on B200, got {d_qk} / {d_v}")
    if d_qk % 8 or d_v % 8:
      raise NotImplementedError(f"head dims must be multiples of 8 (16-byte rows), got {d_qk} / {d_v}")
    q_seg = kv_seg = None
    if segment_ids is not None:
      q_seg = torch.as_tensor(segment_ids.q, device=q.device).to(torch.int32)
      kv_seg = torch.as_tensor(segment_ids.kv, device=q.device).to(torch.int32)
      if q_seg.dim() == 1:
        q_seg = q_seg[None].expand(q.shape[0], -1)
        kv_seg = kv_seg[None].expand(q.shape[0], -1)
      if q_seg.shape != (q.shape[0], q_len) or kv_seg.shape != (q.shape[0], kv_len):
        raise ValueError(f"segment id shapes {tuple(q_seg.shape)}, {tuple(kv_seg.shape)} do not match q/kv")
      q_seg, kv_seg = q_seg.contiguous(), kv_seg.contiguous()
    hq = q.shape[1]
    if sinks is not None:
      sinks = torch.as_tensor(sinks, device=q.device)
      if sinks.shape != (hq,):
        raise ValueError(f"sinks.shape={tuple(sinks.shape)} != num_q_heads={hq}")
    max_logit = None
    if max_logit_value is not None or self.config.max_logit_const is not None:
      value = max_logit_value if max_logit_value is not None else self.config.max_logit_const
      value = torch.as_tensor(value, dtype=torch.float32, device=q.device)
      if tuple(value.shape) not in ((), (1,), (hq,)):
        raise ValueError(f"max_logit_value should have shape (), (1,) or ({hq},), got {tuple(value.shape)}")
      max_logit = value.reshape(-1).expand(hq).contiguous()
    apply = _function if _function is not None else _SplashFunction.apply
    o, lse, max_logits = apply(q, k, v, q_seg, kv_seg, self, float(logits_scale), sinks, max_logit, int(q_shard))
    if not batched:
      o, lse, max_logits = o[0], lse[0], max_logits[0]
    if save_residuals:
      return o, {"logsumexp": lse, "max_logits": max_logits}
    return o

  def manual_sharding_spec(self, sharding):
    raise NotImplementedError(
        "a shard_map partition spec is a JAX construct; a kernel built with q_seq_shards=n takes the q rows of "
        "shard i through `kernel(q_i, k, v, q_shard=i)`, and tokamax_b200.q_seq_sharding.QSeqShardedSplashAttention "
        "runs one shard per rank of a process group"
    )

  # pytree-style helpers kept for API parity with the reference
  def tree_flatten(self):
    return ((self.fwd_mask_info, self.dkv_mask_info), self.kwargs)

  @classmethod
  def tree_unflatten(cls, kwargs, values):
    fwd_mask_info, dkv_mask_info = values
    dkv_mask_info = MaskInfo(*dkv_mask_info) if dkv_mask_info is not None else None
    return SplashAttentionKernel(MaskInfo(*fwd_mask_info), dkv_mask_info, **kwargs)


# ----------------------------------------------------------------------------------------------
# factories
# ----------------------------------------------------------------------------------------------
def _live_fraction(block_mask) -> float:
  """Share of non-empty blocks in a block_mask table (0 for a mask with no live block)."""
  block_mask = np.asarray(block_mask)
  return float(np.mean(block_mask != 0)) if block_mask.size else 0.0


def _make_splash_attention(
    mask: np.ndarray | mask_lib.Mask,
    *,
    config: SplashConfig | None = None,
    is_mqa: bool,
    save_residuals: bool = False,
    mask_value: float = DEFAULT_MASK_VALUE,
    downcast_smem_data: bool = True,
    partial_mask_blocks_dtype: Any = np.int8,
    q_seq_shards: int,
    repeatable_dq: bool = False,
):
  if len(mask.shape) != 2:
    raise ValueError(f"Unexpected mask shape: {mask.shape}")
  if isinstance(mask, np.ndarray):
    mask = mask_lib.NumpyMask(mask)
  if config is None:
    config = SplashConfig.get_default()
  if q_seq_shards < 1 or (q_seq_shards > 1 and mask.shape[0] % (q_seq_shards * _TILE) != 0):
    raise ValueError(f"q_seq_shards={q_seq_shards} must cut the {mask.shape[0]} q rows into multiples of {_TILE}")
  process_fn = partial(
      mask_info_lib.process_mask,
      downcast_smem_data=downcast_smem_data,
      partial_mask_blocks_dtype=partial_mask_blocks_dtype,
      q_seq_shards=q_seq_shards,
  )
  fwd_mask_info, mask_function_fwd = process_fn(mask, (config.block_q, config.block_kv))
  fwd_mask_sparsity = (
      _live_fraction(fwd_mask_info.block_mask) if fwd_mask_info.block_mask is not None else 1.0
  )
  dkv_mask_info = None
  dkv_mask_sparsity = 1.0
  if config.has_backward_blocks:
    dkv_mask_info, mask_function_dkv = process_fn(
        mask,
        (config.block_q_dkv, config.block_kv_dkv),
        is_dkv=True,
        return_dynamic_grid=config.dq_reduction_steps == 3,
    )
    assert (mask_function_fwd is None) == (mask_function_dkv is None)
    if dkv_mask_info.block_mask is not None:
      dkv_mask_sparsity = _live_fraction(dkv_mask_info.block_mask)
  rule = mask.interval_rule if mask_function_fwd is not None else None
  return SplashAttentionKernel(
      fwd_mask_info,
      dkv_mask_info,
      config=config,
      is_mqa=is_mqa,
      save_residuals=save_residuals,
      mask_value=mask_value,
      mask_function=mask_function_fwd,
      mask_function_rule=rule,
      mask_shape=tuple(mask.shape),
      fwd_mask_sparsity=fwd_mask_sparsity,
      dkv_mask_sparsity=dkv_mask_sparsity,
      repeatable_dq=repeatable_dq,
      q_seq_shards=q_seq_shards,
  )


def _make_dynamic_splash_attention(
    mask,
    *,
    mesh=None,
    mask_spec=None,
    config: SplashConfig | None = None,
    is_mqa: bool,
    save_residuals: bool = False,
    mask_value: float = DEFAULT_MASK_VALUE,
    downcast_smem_data: bool = True,
    partial_mask_blocks_dtype: Any = np.int8,
    repeatable_dq: bool = False,
):
  """Kernel for a mask that is data (a bool array / tensor) rather than a static object."""
  if (mesh is not None) != (mask_spec is not None):
    raise ValueError("Either both or neither of mesh and mask_spec must be specified.")
  if mesh is not None:
    raise NotImplementedError("mesh / mask_spec belong to shard_map; not applicable on B200")
  if len(mask.shape) != 2:
    raise ValueError(f"Unexpected mask shape: {mask.shape}")
  if config is None:
    config = SplashConfig.get_default()
  config = dataclasses.replace(config, dq_reduction_steps=3)
  if isinstance(mask, torch.Tensor) and mask.is_cuda:
    # Device path: nothing of the mask goes through the host (the kernel object snapshots the
    # tensor it is given; build a new one, which is cheap, when the mask changes).
    return SplashAttentionKernel(
        None, None, dynamic_mask=mask, config=config, is_mqa=is_mqa, save_residuals=save_residuals,
        mask_value=mask_value, mask_function=None, mask_function_rule=None, mask_shape=tuple(mask.shape),
        fwd_mask_sparsity=1.0, dkv_mask_sparsity=1.0, repeatable_dq=repeatable_dq)
  process = partial(
      mask_info_lib._process_dynamic_mask,  # pylint: disable=protected-access
      downcast_smem_data=downcast_smem_data,
      partial_mask_blocks_dtype=partial_mask_blocks_dtype,
  )
  fwd_mask_info = process(mask, (config.block_q, config.block_kv), is_dkv=False)
  dkv_mask_info = None
  if config.has_backward_blocks:
    dkv_mask_info = process(mask, (config.block_q_dkv, config.block_kv_dkv), is_dkv=True)
  return SplashAttentionKernel(
      fwd_mask_info,
      dkv_mask_info,
      config=config,
      is_mqa=is_mqa,
      save_residuals=save_residuals,
      mask_value=mask_value,
      mask_function=None,
      mask_function_rule=None,
      mask_shape=tuple(mask.shape),
      fwd_mask_sparsity=1.0,
      dkv_mask_sparsity=1.0,
      repeatable_dq=repeatable_dq,
  )


make_splash_mha = partial(_make_splash_attention, is_mqa=False)
make_splash_mqa = partial(_make_splash_attention, is_mqa=True)

make_splash_mha_single_device = partial(make_splash_mha, q_seq_shards=1)
make_splash_mqa_single_device = partial(make_splash_mqa, q_seq_shards=1)

make_dynamic_splash_mqa = partial(_make_dynamic_splash_attention, is_mqa=True)
make_dynamic_splash_mha = partial(_make_dynamic_splash_attention, is_mqa=False)
