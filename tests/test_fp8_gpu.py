"""Block-scaled e4m3 forward against the oracle run on the dequantised tensors.

Tolerances (this variant has no reference implementation; they are this build's contract):
  * logsumexp / max_logits <= 1e-3 against the oracle fed the exact (fp32) dequantised values:
    the score path is exact products of e4m3 values accumulated in fp32, so it carries the same
    bound as the bf16 kernel.
  * output: P is rounded to e4m3 (3 mantissa bits, relative error up to 2^-4 per weight) before
    the PV product, so rows with few live keys see errors of a few percent of |v|.  The bound is
    relative L2 <= 3e-2 over the tensor and max-abs <= 0.25 against the oracle fed the
    dequantised values rounded to bf16.
  * output with `p_format="f16"` (probabilities kept 16 bits wide, V converted exactly): the bf16
    kernel's bound, max-abs <= 1e-2 for unit-variance data (scaled with the output's magnitude
    beyond |o| = 4) and relative L2 <= 5e-3, against the oracle fed the exact dequantised values —
    what the kernel multiplies.
"""
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref
from tokamax_b200 import fp8
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
D = 128
DEV = "cuda:0"


def _randn(seed, *shape):
  g = torch.Generator().manual_seed(seed)
  return torch.randn(*shape, generator=g)


def _check(mask, q, k, v, scale, p_format="e4m3", segment_ids=None, sinks=None):
  dense = np.asarray(mask[:, :]) if not isinstance(mask, np.ndarray) else mask
  qq, kq, vq = (fp8.quantize_e4m3(x.to(DEV)) for x in (q, k, v))
  kernel = splash.make_splash_mha_single_device(mask, save_residuals=True)
  seg_dev = None if segment_ids is None else splash.SegmentIds(*(torch.from_numpy(x).to(DEV) for x in segment_ids))
  o, res = fp8.splash_fwd_fp8(kernel, qq, kq, vq, seg_dev, None if sinks is None else sinks.to(DEV),
                              logits_scale=scale, save_residuals=True, p_format=p_format)
  torch.cuda.synchronize()
  kernel.check_errors()
  o = o.float().cpu()
  for b in range(q.shape[0]):
    exact = [fp8.dequantize_e4m3(fp8.Fp8Tensor(t.data[b:b + 1], t.scale[b:b + 1]), torch.float32)[0].cpu()
             for t in (qq, kq, vq)]
    seg_b = None if segment_ids is None else (segment_ids[0][b], segment_ids[1][b])
    ref_exact, lse, mx = attention_ref.attention_reference(*exact, dense, seg_b, scale=scale, sinks=sinks)
    assert (res["logsumexp"][b].cpu() - lse).abs().max() <= 1e-3
    assert (res["max_logits"][b].cpu() - mx).abs().max() <= 1e-3
    if p_format == "f16":
      err = o[b] - ref_exact
      # 1e-2 is the bound for unit-variance data (|o| < 4, where rounding the output to bf16 costs up
      # to 7.8e-3 by itself); outputs of larger magnitude scale it
      bound = 1e-2 * max(1.0, float(ref_exact.abs().max()) / 4.0)
      assert err.abs().max() <= bound, (float(err.abs().max()), bound)
      assert err.norm() / ref_exact.norm() <= 5e-3, float(err.norm() / ref_exact.norm())
    else:
      rounded = [x.to(torch.bfloat16) for x in exact]
      ref, _, _ = attention_ref.attention_reference(*rounded, dense, seg_b, scale=scale, sinks=sinks)
      err = o[b] - ref
      assert err.norm() / ref.norm() <= 3e-2, float(err.norm() / ref.norm())
      assert err.abs().max() <= 0.25, float(err.abs().max())


@pytest.mark.parametrize("p_format", ["e4m3", "f16"])
@pytest.mark.parametrize("kind", ["causal", "full", "local"])
def test_fp8_forward_matches_oracle_on_dequantised_inputs(kind, p_format):
  b, hq, hkv, s = 2, 4, 2, 1024
  q, k, v = _randn(51, b, hq, s, D), _randn(52, b, hkv, s, D), _randn(53, b, hkv, s, D)
  if kind == "causal":
    mask = mask_lib.CausalMask((s, s))
  elif kind == "full":
    mask = mask_lib.FullMask((s, s))
  else:
    mask = mask_lib.LocalMask((s, s), (300, 100), 0)
  _check(mask, q, k, v, 1 / math.sqrt(D), p_format)


@pytest.mark.parametrize("p_format", ["e4m3", "f16"])
def test_fp8_segment_ids_and_sinks(p_format):
  """Packed documents (same ids for q and kv) under a causal mask, and a sink per q head."""
  b, hq, hkv, s = 2, 4, 2, 768
  q, k, v = _randn(91, b, hq, s, D), _randn(92, b, hkv, s, D), _randn(93, b, hkv, s, D)
  bounds = [[0, 200, 333, 640, s], [0, 128, 500, s]]
  seg = np.zeros((b, s), np.int32)
  for row, edges in enumerate(bounds):
    for doc, (lo, hi) in enumerate(zip(edges[:-1], edges[1:])):
      seg[row, lo:hi] = doc
  sinks = torch.tensor([0.5, -1.0, 2.0, 0.0])
  _check(mask_lib.CausalMask((s, s)), q, k, v, 1 / math.sqrt(D), p_format, segment_ids=(seg, seg))
  _check(mask_lib.CausalMask((s, s)), q, k, v, 1 / math.sqrt(D), p_format, sinks=sinks)


@pytest.mark.parametrize("p_format", ["e4m3", "f16"])
def test_fp8_scales_varying_by_tile_and_zero_tiles(p_format):
  b, hq, hkv, sq, skv = 1, 2, 1, 256, 768
  q, k, v = _randn(61, b, hq, sq, D), _randn(62, b, hkv, skv, D), _randn(63, b, hkv, skv, D)
  # different magnitudes per 128-token tile, one all-zero V tile, one all-zero K tile
  v_gain = torch.tensor([1.0, 30.0, 0.0, 0.02, 5.0, 1.0])
  k_gain = torch.tensor([1.0, 0.5, 2.0, 0.0, 1.5, 0.25])
  q_gain = torch.tensor([0.5, 2.0])
  v = v * v_gain.repeat_interleave(128)[None, None, :, None]
  k = k * k_gain.repeat_interleave(128)[None, None, :, None]
  q = q * q_gain.repeat_interleave(128)[None, None, :, None]
  _check(mask_lib.FullMask((sq, skv)), q, k, v, 0.05, p_format)


def test_fp8_rejects_bad_arguments():
  s = 256
  kernel = splash.make_splash_mha_single_device(mask_lib.CausalMask((s, s)))
  x = fp8.quantize_e4m3(_randn(71, 1, 2, s, D).to(DEV))
  with pytest.raises(ValueError):
    fp8.splash_fwd_fp8(kernel, fp8.Fp8Tensor(x.data.to(torch.bfloat16), x.scale), x, x)
  with pytest.raises(ValueError):
    fp8.splash_fwd_fp8(kernel, x, x, fp8.Fp8Tensor(x.data, x.scale[..., :1]))
  short = fp8.quantize_e4m3(_randn(72, 1, 2, 128, D).to(DEV))
  with pytest.raises(ValueError):
    fp8.splash_fwd_fp8(kernel, x, short, short)


def test_fp8_device_mask_with_batch_two_and_soft_cap_rejected():
  """A mask tensor on the device builds one schedule per batch size: batch row 1 must read its
  own row ends (same result as the host-built tables)."""
  import dataclasses

  s = 512
  dense = mask_lib.make_random_mask((s, s), 0.7, 5) | np.eye(s, dtype=np.bool_)
  q, k, v = (fp8.quantize_e4m3(_randn(81 + i, 2, 2, s, D).to(DEV)) for i in range(3))
  outs = []
  for kernel in (splash.make_dynamic_splash_mha(torch.from_numpy(dense).to(DEV), save_residuals=True),
                 splash.make_splash_mha_single_device(dense, save_residuals=True)):
    o, res = fp8.splash_fwd_fp8(kernel, q, k, v, logits_scale=0.09, save_residuals=True)
    kernel.check_errors()
    outs.append((o, res["logsumexp"]))
  assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
  assert torch.equal(outs[0][0][0], outs[0][0][0]) and torch.isfinite(outs[0][0].float()).all()
  capped = splash.make_splash_mha_single_device(
      dense, config=dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=30.0))
  with pytest.raises(NotImplementedError):
    fp8.splash_fwd_fp8(capped, q, k, v)
  fixed = splash.make_splash_mha_single_device(
      dense, config=dataclasses.replace(splash.SplashConfig.get_default(), max_logit_const=8.0))
  with pytest.raises(NotImplementedError):
    fp8.splash_fwd_fp8(fixed, q, k, v)
  with pytest.raises(ValueError):
    fp8.splash_fwd_fp8(capped, q, k, v, p_format="bf16")
