"""Block-scaled e4m3 forward (inference prefill) on the splash tables.

The reference's splash path takes bf16 / f32 only (`pallas_mosaic_tpu_common.py:40-42`;
quantised inputs are dequantised before they reach it, `tokamax/_src/quantization.py:75-78`), so
this entry has no counterpart there.  Its contract is the bf16 forward on the dequantised
tensors: ``o ~= splash(dequant(q), dequant(k), dequant(v))``.

Storage: ``float8_e4m3fn`` values in ``[B, H, S, D]`` plus one fp32 scale per (batch, head,
128-token tile), ``[B, H, S / 128]``; ``real = stored * scale`` and ``scale = amax / 448``.
"""
from __future__ import annotations

import ctypes as C
from typing import NamedTuple

import torch

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as _k

E4M3_MAX = 448.0
SCALE_TILE = 128


class Fp8Tensor(NamedTuple):
  """e4m3 values `[B, H, S, D]` with fp32 scales `[B, H, S / 128]`."""
  data: torch.Tensor
  scale: torch.Tensor


def quantize_e4m3(x: torch.Tensor) -> Fp8Tensor:
  """`scale = amax / 448` per (batch, head, 128-token tile); values rounded to nearest e4m3."""
  if x.dim() != 4 or x.shape[2] % SCALE_TILE != 0:
    raise ValueError(f"expected [B, H, S, D] with S a multiple of {SCALE_TILE}, got {tuple(x.shape)}")
  b, h, s, d = x.shape
  xf = x.float().reshape(b, h, s // SCALE_TILE, SCALE_TILE * d)
  amax = xf.abs().amax(dim=-1)
  scale = amax / E4M3_MAX
  safe = torch.where(scale > 0, scale, torch.ones_like(scale))
  q = (xf / safe[..., None]).clamp_(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
  return Fp8Tensor(q.reshape(b, h, s, d), scale.contiguous())


def dequantize_e4m3(t: Fp8Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
  """`stored * scale`, rounded once to ``dtype`` (what the bf16 reference run is fed)."""
  b, h, s, d = t.data.shape
  x = t.data.float().reshape(b, h, s // SCALE_TILE, SCALE_TILE, d) * t.scale[..., None, None]
  return x.reshape(b, h, s, d).to(dtype)


def _fp8_desc(t: torch.Tensor) -> _native.SplashTensor:
  d = _k._tensor_desc(t)  # pylint: disable=protected-access
  d.dtype = 2  # SPLASH_F8E4M3
  return d


def splash_fwd_fp8(kernel: _k.SplashAttentionKernel, q: Fp8Tensor, k: Fp8Tensor, v: Fp8Tensor,
                   segment_ids: _k.SegmentIds | None = None, sinks: torch.Tensor | None = None, *,
                   logits_scale: float = 1.0, save_residuals: bool = False, p_format: str = "e4m3"):
  """Forward only: bf16 `o [B, Hq, S, D]` (and logsumexp / max_logits of the dequantised logits).

  `kernel` supplies the mask tables (`make_splash_mha(mask, ...)`).  `segment_ids` (`[B, S]` int32
  each) and `sinks` (`[Hq]`) mean what they mean for the bf16 kernel; soft-capping and a fixed
  maximum are not taken here.

  `p_format`: ``"e4m3"`` rounds the probabilities to e4m3 for p v (fastest; the output is within a
  few percent of the bf16 forward on the dequantised tensors: relative L2 <= 3e-2).  ``"f16"`` keeps
  them 16 bits wide — q k^T still runs on the e4m3 tiles, V tiles are converted to f16 on chip — and
  meets the bf16 forward's bound (max-abs <= 1e-2).
  """
  if p_format not in ("e4m3", "f16"):
    raise ValueError(f"p_format must be 'e4m3' or 'f16', got {p_format!r}")
  for name, t in (("q", q), ("k", k), ("v", v)):
    if t.data.dtype != torch.float8_e4m3fn or t.scale.dtype != torch.float32:
      raise ValueError(f"{name}: expected float8_e4m3fn values with float32 scales")
    if t.data.dim() != 4 or t.scale.shape != (*t.data.shape[:2], t.data.shape[2] // SCALE_TILE):
      raise ValueError(f"{name}: values {tuple(t.data.shape)} / scales {tuple(t.scale.shape)} do not match")
  qd, kd, vd = (t.data.contiguous() for t in (q, k, v))
  qs, ks, vs = (t.scale.contiguous() for t in (q, k, v))
  _k._require_cuda(qd)  # pylint: disable=protected-access
  b, hq, sq, d = qd.shape
  if d != 128 or kd.shape[-1] != 128 or vd.shape[-1] != 128:
    raise NotImplementedError("only head_dim 128 is built on B200")
  if (sq, kd.shape[2]) != tuple(kernel.mask_shape) or vd.shape != kd.shape:
    raise ValueError(f"shapes q {tuple(qd.shape)}, k {tuple(kd.shape)}, v {tuple(vd.shape)} do not match the "
                     f"mask {kernel.mask_shape}")
  if kd.shape[1] == 0 or hq % kd.shape[1] != 0:
    raise ValueError(f"q heads ({hq}) must be a multiple of kv heads ({kd.shape[1]})")
  if kernel.config.attn_logits_soft_cap is not None:
    raise NotImplementedError("attn_logits_soft_cap is not built for the e4m3 forward")
  if kernel.config.max_logit_const is not None:
    raise NotImplementedError("a fixed maximum is not built for the e4m3 forward")
  q_seg = kv_seg = None
  if segment_ids is not None:
    q_seg, kv_seg = (torch.as_tensor(x, device=qd.device).to(torch.int32).contiguous() for x in segment_ids)
    if q_seg.shape != (b, sq) or kv_seg.shape != (b, kd.shape[2]):
      raise ValueError(f"segment ids {tuple(q_seg.shape)} / {tuple(kv_seg.shape)} do not match q / k")
  if sinks is not None and tuple(sinks.shape) != (hq,):
    raise ValueError(f"sinks must have shape ({hq},), got {tuple(sinks.shape)}")
  tables = kernel._tables(qd.device, b)  # pylint: disable=protected-access  (device masks: one table per batch size)
  o = torch.empty((b, hq, sq, d), dtype=torch.bfloat16, device=qd.device)
  lse = torch.empty((b, hq, sq), dtype=torch.float32, device=qd.device)
  max_logits = torch.empty((b, hq, sq), dtype=torch.float32, device=qd.device)
  args = _native.SplashFwdFp8Args()
  base = args.base
  base.q, base.k, base.v = map(_fp8_desc, (qd, kd, vd))
  base.o = _k._tensor_desc(o)  # pylint: disable=protected-access
  base.logsumexp = lse.data_ptr()
  base.max_logits = max_logits.data_ptr()
  base.q_sequence = tables.q_sequence.data_ptr() if tables.q_sequence is not None else None
  base.sched = tables.fwd
  keep = []
  if q_seg is not None:
    base.q_segment_ids, base.kv_segment_ids = q_seg.data_ptr(), kv_seg.data_ptr()
    if not tables.fwd.row_end:  # device-built schedules are not filtered further
      base.sched, ws = _k._segment_schedule(tables.fwd, 0, q_seg, kv_seg, sq, kd.shape[2])  # pylint: disable=protected-access
      keep.append(ws)
  sinks_f32 = None if sinks is None else sinks.detach().to(device=qd.device, dtype=torch.float32).contiguous()
  base.sinks = None if sinks_f32 is None else sinks_f32.data_ptr()
  base.mask_fn = _k._mask_fn_struct(kernel.mask_function_rule)  # pylint: disable=protected-access
  base.scale = float(logits_scale)
  base.mask_value = max(kernel.mask_value, -3.0e38)
  base.error_record = tables.error_record.data_ptr()
  args.q_scale, args.k_scale, args.v_scale = qs.data_ptr(), ks.data_ptr(), vs.data_ptr()
  args.flags = _native.FP8_P_F16 if p_format == "f16" else 0
  stream = torch.cuda.current_stream(qd.device).cuda_stream
  with torch.cuda.device(qd.device):
    _native.check(_native.lib().splash_fwd_fp8(C.byref(args), C.c_void_p(stream)), "splash_fwd_fp8")
  for t in keep + [q_seg, kv_seg, sinks_f32]:
    if t is not None:
      t.record_stream(torch.cuda.current_stream(qd.device))
  if save_residuals:
    return o, {"logsumexp": lse, "max_logits": max_logits}
  return o
