"""Rows whose keys are all masked — in the first tiles they meet, or everywhere.

Two cases the block-sparse walk creates and the dense oracle does not see:
  * a row of a live 128x128 tile that has no live key in that tile (late rows of a local window
    start this way): its running maximum must not be taken from masked logits;
  * a row with no live key at all: the kernels return zeros, logsumexp = max_logits = mask value,
    and such rows contribute nothing to dK / dV.  (The reference leaves these rows undefined: its
    kernel averages V over the visited blocks, its dense oracle over every key.)
The scale sweep matters: before the running maximum had a floor, whether such rows came out
right depended on how masked_logit * scale happened to round.
"""
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


def _inputs(seed, hq, hkv, sq, skv):
  g = torch.Generator().manual_seed(seed)
  mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)
  return mk(1, hq, sq, D), mk(1, hkv, skv, D), mk(1, hkv, skv, D), mk(1, hq, sq, D)


def _rel(a, ref):
  return ((a.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-20)).item()


@pytest.mark.parametrize("scale", [0.03, 0.05, 1 / math.sqrt(D), 0.1, 0.3, 1.0])
def test_rows_masked_in_their_first_tile(scale):
  s = 768
  mask = mask_lib.LocalMask((s, s), (200, 60), 0)  # late rows start in a tile that holds none of their keys
  dense = np.asarray(mask[:, :])
  q, k, v, do = _inputs(81, 4, 2, s, s)
  qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
  kernel = splash.make_splash_mha_single_device(mask, save_residuals=True)
  out, res = kernel(qd, kd, vd, logits_scale=scale)
  out.backward(do.to(DEV))
  kernel.check_errors()
  ro, rlse, _, rdq, rdk, rdv = attention_ref.fwd_bwd(q, k, v, do, dense, None, scale=scale)
  assert torch.isfinite(out.float()).all()
  assert ((out.float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (res["logsumexp"].cpu() - rlse).abs().max() <= 1e-3
  for got, ref in ((qd.grad, rdq), (kd.grad, rdk), (vd.grad, rdv)):
    assert _rel(got, ref) <= 1e-2


@pytest.mark.parametrize("scale", [0.05, 1 / math.sqrt(D), 0.25])
def test_rows_with_no_live_key_anywhere(scale):
  sq, skv = 384, 512
  dense = mask_lib.make_random_mask((sq, skv), 0.4, 9)
  dead = np.r_[3, 100:140, 383]
  dense[dead] = False
  alive = np.setdiff1d(np.arange(sq), dead)
  assert dense[alive].any(axis=1).all()
  q, k, v, do = _inputs(82, 2, 1, sq, skv)
  do[:, :, dead] = 0  # the oracle spreads dead rows uniformly over all keys; keep that out of dK / dV
  qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
  kernel = splash.make_splash_mha_single_device(dense, save_residuals=True)
  out, res = kernel(qd, kd, vd, logits_scale=scale)
  out.backward(do.to(DEV))
  kernel.check_errors()
  ro, rlse, _, rdq, rdk, rdv = attention_ref.fwd_bwd(q, k, v, do, dense, None, scale=scale)
  o = out.float().cpu()
  assert torch.count_nonzero(o[:, :, dead]) == 0
  assert (res["logsumexp"].cpu()[:, :, dead] < -1e37).all() and (res["max_logits"].cpu()[:, :, dead] < -1e37).all()
  # peaky rows reach |o| > 2, where half a bf16 ulp alone is 7.8e-3: atol + rtol * |ref| as the reference's tests
  assert ((o[:, :, alive] - ro[:, :, alive]).abs() <= 1e-2 + 4e-3 * ro[:, :, alive].abs()).all()
  assert (res["logsumexp"].cpu()[:, :, alive] - rlse[:, :, alive]).abs().max() <= 1e-3
  dq = qd.grad.float().cpu()
  assert torch.count_nonzero(dq[:, :, dead]) == 0
  assert _rel(dq[:, :, alive], rdq[:, :, alive]) <= 1e-2
  assert _rel(kd.grad, rdk) <= 1e-2 and _rel(vd.grad, rdv) <= 1e-2
