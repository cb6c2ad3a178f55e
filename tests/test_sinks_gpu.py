"""Attention sinks and the fixed maximum (`max_logit_value` / `max_logit_const`) against the oracle.

Reference: splash_attention_kernel.py:363-395 (initial m / l), :440-470 (fixed maximum),
:1928-1935 (dsinks); base.py:96-104, :166-172.
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
SCALE = 1 / math.sqrt(D)


def _inputs(seed, b, hq, hkv, s):
  g = torch.Generator().manual_seed(seed)
  mk = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)
  return mk(b, hq, s, D), mk(b, hkv, s, D), mk(b, hkv, s, D), mk(b, hq, s, D), torch.randn(hq, generator=g) * 2


def _rel(a, ref):
  return ((a.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-20)).item()


def _oracle(q, k, v, do, dense, sinks):
  outs = []
  for b in range(q.shape[0]):
    o, lse, mx = attention_ref.attention_reference(q[b], k[b], v[b], dense, scale=SCALE, sinks=sinks)
    o_st = o.to(torch.bfloat16)
    dq, dk, dv = attention_ref.attention_reference_vjp(do[b], q[b], k[b], v[b], dense, None, o_st, lse, scale=SCALE)
    ds = attention_ref.sinks_vjp(do[b], o_st, lse, sinks) if sinks is not None else torch.zeros(q.shape[1])
    outs.append((o, lse, mx, dq, dk, dv, ds))
  stacked = [torch.stack([t[i] for t in outs]) for i in range(7)]
  stacked[6] = stacked[6].sum(0)  # sinks are shared by the batch rows
  return stacked


@pytest.mark.parametrize("kind", ["causal", "local"])
def test_sinks_forward_backward(kind):
  b, hq, hkv, s = 2, 4, 2, 384
  q, k, v, do, sinks = _inputs(91, b, hq, hkv, s)
  mask = mask_lib.CausalMask((s, s)) if kind == "causal" else mask_lib.LocalMask((s, s), (150, 20), 0)
  dense = np.asarray(mask[:, :])
  kernel = splash.make_splash_mha_single_device(mask, save_residuals=True)
  qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
  sd = sinks.to(DEV).requires_grad_(True)
  out, res = kernel(qd, kd, vd, None, sd, logits_scale=SCALE)
  out.backward(do.to(DEV))
  kernel.check_errors()
  ro, rlse, rmx, rdq, rdk, rdv, rds = _oracle(q, k, v, do, dense, sinks)
  assert ((out.float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (res["logsumexp"].cpu() - rlse).abs().max() <= 1e-3
  assert (res["max_logits"].cpu() - rmx).abs().max() <= 1e-3
  for got, ref in ((qd.grad, rdq), (kd.grad, rdk), (vd.grad, rdv), (sd.grad, rds)):
    assert _rel(got, ref) <= 1e-2
  # the sink takes weight away from the keys: row sums of the implied probabilities drop below 1
  no_sink, res0 = kernel(qd.detach(), kd.detach(), vd.detach(), logits_scale=SCALE)
  assert (res["logsumexp"] >= res0["logsumexp"]).all()


@pytest.mark.parametrize("how", ["scalar", "per_head", "config_const"])
def test_fixed_maximum_changes_nothing_but_max_logits(how):
  b, hq, hkv, s = 1, 4, 2, 512
  q, k, v, do, _ = _inputs(92, b, hq, hkv, s)
  mask = mask_lib.CausalMask((s, s))
  base_kernel = splash.make_splash_mha_single_device(mask, save_residuals=True)
  kw, kernel = {}, base_kernel
  per_head = torch.tensor([6.0, 7.5, 9.0, 12.0])
  if how == "scalar":
    kw = dict(max_logit_value=torch.tensor(8.0))
    expect = torch.full((hq,), 8.0)
  elif how == "per_head":
    kw = dict(max_logit_value=per_head.to(DEV))
    expect = per_head
  else:
    kernel = splash.make_splash_mha_single_device(mask, save_residuals=True,
                                                  config=dataclasses.replace(splash.SplashConfig.get_default(), max_logit_const=10.0))
    expect = torch.full((hq,), 10.0)
  qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
  out, res = kernel(qd, kd, vd, logits_scale=SCALE, **kw)
  out.backward(do.to(DEV))
  kernel.check_errors()
  ro, rlse, _, rdq, rdk, rdv, _ = _oracle(q, k, v, do, np.asarray(mask[:, :]), None)
  assert ((out.float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (res["logsumexp"].cpu() - rlse).abs().max() <= 1e-3
  assert torch.allclose(res["max_logits"].cpu(), expect[None, :, None].expand(b, hq, s), atol=1e-5)
  for got, ref in ((qd.grad, rdq), (kd.grad, rdk), (vd.grad, rdv)):
    assert _rel(got, ref) <= 1e-2


def test_sinks_with_fixed_maximum_and_rows_without_keys():
  hq, hkv, sq, skv = 2, 1, 256, 384
  q, k, v, do, sinks = _inputs(93, 1, hq, hkv, 384)
  q, do = q[:, :, :sq], do[:, :, :sq]
  dense = mask_lib.make_random_mask((sq, skv), 0.5, 3)
  dead = np.r_[7, 200:210]
  dense[dead] = False
  kernel = splash.make_splash_mha_single_device(dense, save_residuals=True)
  out, res = kernel(q.to(DEV), k.to(DEV), v.to(DEV), None, sinks.to(DEV), max_logit_value=torch.tensor(9.0),
                    logits_scale=SCALE)
  kernel.check_errors()
  ro, rlse, _ = attention_ref.attention_reference(q[0], k[0], v[0], dense, scale=SCALE, sinks=sinks)
  alive = np.setdiff1d(np.arange(sq), dead)
  o = out.float().cpu()[0]
  assert ((o[:, alive] - ro[:, alive]).abs() <= 1e-2 + 4e-3 * ro[:, alive].abs()).all()
  assert (res["logsumexp"].cpu()[0][:, alive] - rlse[:, alive]).abs().max() <= 1e-3
  # rows with no live key: the sink is the only term of the softmax
  assert torch.count_nonzero(o[:, dead]) == 0
  assert torch.allclose(res["logsumexp"].cpu()[0][:, dead], sinks[:, None].expand(hq, len(dead)), atol=1e-4)


def test_argument_errors():
  s = 256
  kernel = splash.make_splash_mha_single_device(mask_lib.CausalMask((s, s)),
                                                config=dataclasses.replace(splash.SplashConfig.get_default(), max_logit_const=5.0))
  q, k, v, _, sinks = _inputs(94, 1, 2, 2, s)
  with pytest.raises(ValueError):
    kernel(q.to(DEV), k.to(DEV), v.to(DEV), max_logit_value=torch.tensor(1.0))
  plain = splash.make_splash_mha_single_device(mask_lib.CausalMask((s, s)))
  with pytest.raises(ValueError):
    plain(q.to(DEV), k.to(DEV), v.to(DEV), None, torch.zeros(3))
  with pytest.raises(ValueError):
    plain(q.to(DEV), k.to(DEV), v.to(DEV), max_logit_value=torch.zeros(3))
