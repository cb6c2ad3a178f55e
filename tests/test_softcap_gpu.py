"""attn_logits_soft_cap: logits = cap * tanh(scale * q k^T / cap), forward and backward.

Reference: splash_attention_kernel.py:202-296 (cap, then mask), base.py:92-94 and :159-163 (the
backward chain factor 1 - tanh^2).
"""
import dataclasses
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
D = 128
DEV = "cuda:0"


def _rel(a, ref):
  return ((a.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-20)).item()


@pytest.mark.parametrize("cap,scale,dims", [(30.0, 1 / math.sqrt(D), (D, D)), (8.0, 0.35, (D, D)),
                                            (2.0, 1 / math.sqrt(D), (D, D)), (8.0, 0.2, (192, 128)),
                                            (4.0, 1 / 16, (256, 256))])
@pytest.mark.parametrize("kind", ["causal", "local_segments"])
def test_soft_cap_forward_backward(cap, scale, dims, kind):
  """(128, 128), and the head dims above 128 that run the two-panel kernels."""
  b, hq, hkv, s = 1, 4, 2, 512
  d_qk, d_v = dims
  g = torch.Generator().manual_seed(int(cap * 10) + len(kind) + d_qk)
  mk = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)
  q, k, v, do = mk(b, hq, s, d_qk), mk(b, hkv, s, d_qk), mk(b, hkv, s, d_v), mk(b, hq, s, d_v)
  seg = None
  if kind == "causal":
    mask = mask_lib.CausalMask((s, s))
  else:
    mask = mask_lib.LocalMask((s, s), (200, 0), 0)
    ids = torch.from_numpy(np.repeat(np.arange(4, dtype=np.int32), [100, 156, 56, 200]))
    seg = (ids, ids)
  dense = np.asarray(mask[:, :])
  cfg = dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=cap)
  kernel = splash.make_splash_mha_single_device(mask, config=cfg, save_residuals=True)
  qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
  seg_dev = None if seg is None else splash.SegmentIds(seg[0][None].to(DEV), seg[1][None].to(DEV))
  out, res = kernel(qd, kd, vd, seg_dev, logits_scale=scale)
  out.backward(do.to(DEV))
  kernel.check_errors()
  ro, rlse, rmx = attention_ref.attention_reference(q[0], k[0], v[0], dense, seg, scale=scale,
                                                    attn_logits_soft_cap=cap)
  rdq, rdk, rdv = attention_ref.attention_reference_vjp(do[0], q[0], k[0], v[0], dense, seg, ro.to(torch.bfloat16),
                                                        rlse, scale=scale, attn_logits_soft_cap=cap)
  assert ((out.float().cpu()[0] - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (res["logsumexp"].cpu()[0] - rlse).abs().max() <= 1e-3
  assert (res["max_logits"].cpu()[0] - rmx).abs().max() <= 1e-3
  assert (res["max_logits"] <= cap + 1e-4).all()
  for got, ref in ((qd.grad[0], rdq), (kd.grad[0], rdk), (vd.grad[0], rdv)):
    assert _rel(got, ref) <= 1e-2


def test_soft_cap_changes_the_result_and_rejects_bad_values():
  s = 256
  g = torch.Generator().manual_seed(3)
  q = torch.randn(1, 2, s, D, generator=g).to(torch.bfloat16).to(DEV)
  mask = mask_lib.CausalMask((s, s))
  plain = splash.make_splash_mha_single_device(mask)(q, q, q, logits_scale=0.3)
  cfg = dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=3.0)
  capped = splash.make_splash_mha_single_device(mask, config=cfg)(q, q, q, logits_scale=0.3)
  assert (plain.float() - capped.float()).abs().max() > 0.05
  bad = dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=-1.0)
  with pytest.raises(ValueError):
    splash.make_splash_mha_single_device(mask, config=bad)(q, q, q)
