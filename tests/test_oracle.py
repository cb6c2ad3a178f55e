"""Pins the numeric oracle (oracle/attention_ref.py).

(1) Against the reference's own dense oracle: tests/golden/attention_golden.npz holds the outputs
of the reference's ``attention_reference`` / ``attention_reference_vjp`` (base.py:185-285), run
unmodified with numpy standing in for ``jax.numpy`` (tests/golden/gen_attention_golden.py; JAX is
not installed where the vectors were made, so what differs from a run under XLA is the order of
fp32 summation).  Where a checkout of the reference is at hand (SPLASH_REFERENCE_ROOT) the same
comparison also runs live on further random cases.  (2) Against two independent evaluations: a
float64 numpy softmax attention written from the definition, and torch autograd of the oracle's own
forward for the backward formulas (both the "flash" and the "vanilla" di).
"""
import math
import os
import sys

import numpy as np
import pytest
import torch

from oracle import attention_ref
from oracle import ref_loader
from tokamax_b200 import splash_attention_mask as mask_lib

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import attention_cases  # noqa: E402  pylint: disable=wrong-import-position

ATTENTION_GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_golden.npz"))


def _restated(case, q, k, v, do, mask, seg, sinks, impl):
  """The restatement's outputs for one case, as float32 numpy arrays keyed like the golden file."""
  t = lambda x: None if x is None else torch.from_numpy(np.ascontiguousarray(x))
  o, lse, mx = attention_ref.attention_reference(t(q), t(k), t(v), mask, seg, scale=1.0,
                                                 attn_logits_soft_cap=case["soft_cap"], sinks=t(sinks))
  o_stored = torch.from_numpy(attention_cases.to_bf16(o.numpy()))
  dq, dk, dv = attention_ref.attention_reference_vjp(t(do), t(q), t(k), t(v), mask, seg, o_stored, lse, scale=1.0,
                                                     attn_logits_soft_cap=case["soft_cap"], backward_impl=impl)
  out = {"o": o, "logsumexp": lse, "max_logits": mx, f"{impl}/dq": dq, f"{impl}/dk": dk, f"{impl}/dv": dv}
  if sinks is not None:
    out[f"{impl}/dsinks"] = attention_ref.sinks_vjp(t(do), o_stored, lse, t(sinks))
  return {key: val.numpy() for key, val in out.items()}


def _close(got, want, what):
  assert got.shape == want.shape, (what, got.shape, want.shape)
  # fp32 on both sides; the sums (over up to 128 terms with cancellation) are taken in different orders
  scale = max(1.0, float(np.abs(want).max()))
  assert np.abs(got - want).max() <= 1e-4 * scale, (what, float(np.abs(got - want).max()), scale)


@pytest.mark.parametrize("case", attention_cases.CASES, ids=lambda c: c["name"])
def test_restatement_matches_the_references_own_oracle(case):
  q, k, v, do, mask, seg, sinks = attention_cases.build(case)
  for impl in ("flash", "vanilla") if case["name"] in attention_cases.VANILLA_TOO else ("flash",):
    got = _restated(case, q, k, v, do, mask, seg, sinks, impl)
    for key, value in got.items():
      _close(value, ATTENTION_GOLDEN[f"{case['name']}/{key}"], (case["name"], key))
  stored = [key for key in ATTENTION_GOLDEN.files if key.startswith(case["name"] + "/")]
  assert len(stored) >= 6  # o, logsumexp, max_logits, dq, dk, dv (+ dsinks, + the vanilla set)


@pytest.mark.skipif(not ref_loader.available(), reason="needs a checkout of the reference (SPLASH_REFERENCE_ROOT)")
def test_restatement_matches_the_reference_live_on_random_cases():
  import random

  base = ref_loader.load_reference_base()
  for n in range(25):
    rng = random.Random(n)
    mqa = rng.random() < 0.3
    hkv = 1 if mqa else rng.choice([1, 2, 3])
    case = dict(name=f"live{n}", hq=hkv * rng.choice([1, 2, 4]), hkv=hkv, s=8 * rng.randint(2, 12), t=0,
                d=rng.choice([16, 32, 64]), dv=rng.choice([16, 32, 64]), mask=rng.choice(["causal", "local", "random"]),
                mqa=mqa, segments=rng.random() < 0.4, sinks=rng.random() < 0.4,
                soft_cap=rng.choice([None, None, 3.0, 30.0]), seed=100 + n)
    case["t"] = case["s"] if rng.random() < 0.7 else 8 * rng.randint(2, 12)
    q, k, v, do, mask, seg, sinks = attention_cases.build(case)
    seg_ids = None if seg is None else base.SegmentIds(q=seg[0], kv=seg[1])
    kw = dict(is_mqa=mqa, attn_logits_soft_cap=case["soft_cap"])
    o, res = base.attention_reference(q, k, v, mask, seg_ids, sinks, save_residuals=True, **kw)
    impl = rng.choice(["flash", "vanilla"])
    dq, dk, dv, dsinks = base.attention_reference_vjp(do, q, k, v, mask, seg_ids, sinks, attention_cases.to_bf16(o),
                                                      res["logsumexp"], backward_impl=impl, **kw)
    want = {"o": o, "logsumexp": res["logsumexp"], "max_logits": res["max_logits"], f"{impl}/dq": dq,
            f"{impl}/dk": dk, f"{impl}/dv": dv}
    if dsinks is not None:
      want[f"{impl}/dsinks"] = dsinks
    got = _restated(case, q, k, v, do, mask, seg, sinks, impl)
    assert set(got) == set(want), (case, sorted(got), sorted(want))
    for key in want:
      _close(got[key], np.asarray(want[key], dtype=np.float32), (case, key))


def _numpy_attention(q, k, v, mask, scale):
  q, k, v = (t.double().numpy() for t in (q, k, v))
  group = q.shape[0] // k.shape[0]
  outs, lses = [], []
  for h in range(q.shape[0]):
    logits = (q[h] @ k[h // group].T) * scale
    logits = np.where(mask, logits, -np.inf)
    m = logits.max(-1, keepdims=True)
    e = np.exp(logits - m)
    l = e.sum(-1, keepdims=True)
    outs.append((e / l) @ v[h // group])
    lses.append((m + np.log(l))[:, 0])
  return np.stack(outs), np.stack(lses)


@pytest.mark.parametrize("hq,hkv", [(2, 2), (4, 1), (6, 2)])
def test_forward_matches_float64_definition(hq, hkv):
  g = torch.Generator().manual_seed(hq * 10 + hkv)
  s, t, d = 48, 80, 16
  q, k, v = (torch.randn(h, n, d, generator=g) for h, n in ((hq, s), (hkv, t), (hkv, t)))
  mask = mask_lib.make_causal_mask((s, t), offset=32)
  o, lse, mx = attention_ref.attention_reference(q, k, v, mask, scale=0.3)
  ro, rlse = _numpy_attention(q, k, v, mask, 0.3)
  np.testing.assert_allclose(o.numpy(), ro, rtol=2e-5, atol=2e-6)
  np.testing.assert_allclose(lse.numpy(), rlse, rtol=2e-6, atol=2e-6)
  assert torch.all(mx <= lse + 1e-6)


@pytest.mark.parametrize("impl", ["flash", "vanilla"])
def test_backward_matches_autograd(impl):
  g = torch.Generator().manual_seed(5)
  hq, hkv, s, d = 4, 2, 40, 8
  q = torch.randn(hq, s, d, generator=g, requires_grad=True)
  k = torch.randn(hkv, s, d, generator=g, requires_grad=True)
  v = torch.randn(hkv, s, d, generator=g, requires_grad=True)
  do = torch.randn(hq, s, d, generator=g)
  mask = mask_lib.make_local_attention_mask((s, s), (9, 0))
  seg = torch.from_numpy(np.repeat(np.arange(4, dtype=np.int32), 10))
  o, lse, _ = attention_ref.attention_reference(q, k, v, mask, (seg, seg), scale=0.5)
  o.backward(do)
  dq, dk, dv = attention_ref.attention_reference_vjp(
      do, q.detach(), k.detach(), v.detach(), mask, (seg, seg), o.detach(), lse.detach(), scale=0.5,
      backward_impl=impl)
  torch.testing.assert_close(dq, q.grad, rtol=1e-4, atol=1e-5)
  torch.testing.assert_close(dk, k.grad, rtol=1e-4, atol=1e-5)
  torch.testing.assert_close(dv, v.grad, rtol=1e-4, atol=1e-5)


def test_soft_cap_and_mqa_paths():
  g = torch.Generator().manual_seed(9)
  q = torch.randn(3, 16, 8, generator=g, requires_grad=True)
  k = torch.randn(16, 8, generator=g, requires_grad=True)
  v = torch.randn(16, 8, generator=g, requires_grad=True)
  do = torch.randn(3, 16, 8, generator=g)
  mask = mask_lib.make_causal_mask((16, 16))
  o, lse, _ = attention_ref.attention_reference(q, k, v, mask, scale=1.0, attn_logits_soft_cap=5.0)
  o.backward(do)
  dq, dk, dv = attention_ref.attention_reference_vjp(do, q.detach(), k.detach(), v.detach(), mask, None,
                                                     o.detach(), lse.detach(), attn_logits_soft_cap=5.0)
  torch.testing.assert_close(dq, q.grad, rtol=1e-4, atol=1e-5)
  torch.testing.assert_close(dk, k.grad, rtol=1e-4, atol=1e-5)
  torch.testing.assert_close(dv, v.grad, rtol=1e-4, atol=1e-5)
  assert dk.shape == k.shape


def test_masked_rows_use_the_finite_mask_value():
  """A fully masked row averages V (the reference's finite mask value, base.py:28-30,99)."""
  q = torch.zeros(1, 4, 8)
  k = torch.zeros(1, 4, 8)
  v = torch.arange(32, dtype=torch.float32).view(1, 4, 8)
  mask = np.zeros((4, 4), bool)
  mask[1:] = np.tril(np.ones((4, 4), bool))[1:]
  o, lse, mx = attention_ref.attention_reference(q, k, v, mask)
  torch.testing.assert_close(o[0, 0], v[0].mean(0))
  assert mx[0, 0].item() == pytest.approx(attention_ref.DEFAULT_MASK_VALUE)


def test_sinks_forward_and_gradient():
  """Sinks (base.py:96-104, :166-172): float64 definition with one extra value-less key per head,
  and autograd of the oracle's own forward for dq / dk / dv / dsinks."""
  g = torch.Generator().manual_seed(11)
  hq, hkv, s, d = 4, 2, 24, 8
  q = torch.randn(hq, s, d, generator=g, requires_grad=True)
  k = torch.randn(hkv, s, d, generator=g, requires_grad=True)
  v = torch.randn(hkv, s, d, generator=g, requires_grad=True)
  sinks = (torch.randn(hq, generator=g) * 2).requires_grad_(True)
  do = torch.randn(hq, s, d, generator=g)
  mask = mask_lib.make_causal_mask((s, s))
  o, lse, mx = attention_ref.attention_reference(q, k, v, mask, scale=0.4, sinks=sinks)
  # definition: softmax over the live keys plus the sink, whose value is zero
  for h in range(hq):
    logits = (q[h].detach().double() @ k[h // 2].detach().double().T) * 0.4
    logits = torch.where(torch.from_numpy(mask), logits, torch.tensor(-math.inf, dtype=torch.float64))
    full = torch.cat([logits, sinks[h].detach().double().expand(s, 1)], dim=1)
    p = torch.softmax(full, dim=-1)[:, :-1]
    np.testing.assert_allclose(o[h].detach().numpy(), (p @ v[h // 2].detach().double()).numpy(), rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(lse[h].detach().numpy(), torch.logsumexp(full, dim=-1).numpy(), rtol=2e-6, atol=2e-6)
    assert torch.all(mx[h] >= sinks[h] - 1e-6)
  o.backward(do)
  dq, dk, dv = attention_ref.attention_reference_vjp(do, q.detach(), k.detach(), v.detach(), mask, None,
                                                     o.detach(), lse.detach(), scale=0.4)
  dsinks = attention_ref.sinks_vjp(do, o.detach(), lse.detach(), sinks.detach())
  for got, ref in ((dq, q.grad), (dk, k.grad), (dv, v.grad), (dsinks, sinks.grad)):
    np.testing.assert_allclose(got.numpy(), ref.numpy(), rtol=2e-4, atol=2e-5)
