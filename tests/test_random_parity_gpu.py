"""Seeded random sweep over the forward / backward arguments against the oracle.

The reference's kernel test draws its cases with hypothesis (splash_attention_kernel_test.py:
233-260: sequence lengths, q / kv heads, head dims, mask kinds, segment ids, soft cap); this file
draws the same kinds of cases from a fixed seed: batch, grouped heads, unequal q / kv lengths, head
dims from 8 to 256 (q k and v independently), every mask kind, packed segments, soft cap, both
backward forms.  Bounds: o within 1e-2 + 4e-3 |o|, logsumexp 1e-3, gradients relative L2 1e-2.
"""
import dataclasses
import math
import random

import numpy as np
import pytest
import torch

from oracle import attention_ref
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
CASES_PER_SEED = 30


def _rel(a, ref):
  return ((a.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-20)).item()


def _draw(rng):
  b = rng.choice([1, 2])
  hkv = rng.choice([1, 2, 3])
  hq = hkv * rng.choice([1, 2, 4])
  sq = 128 * rng.randint(1, 6)
  skv = sq if rng.random() < 0.6 else 128 * rng.randint(1, 6)
  if rng.random() < 0.35:  # head dims above 128 on at least one side
    d_qk, d_v = 8 * rng.randint(17, 32), 8 * rng.randint(1, 32)
    if rng.random() < 0.3:
      d_qk, d_v = 8 * rng.randint(1, 16), 8 * rng.randint(17, 32)
  else:
    d_qk = rng.choice([128, 128, 64, 8 * rng.randint(1, 16)])
    d_v = rng.choice([d_qk, 128, 8 * rng.randint(1, 16)])
  kind = rng.choice(["causal", "local", "chunked", "table", "full", "composed"])
  if kind == "causal":
    mask = mask_lib.CausalMask((sq, skv), offset=rng.choice([0, 0, skv - sq, 37]))
  elif kind == "local":
    mask = mask_lib.LocalMask((sq, skv), (rng.choice([None, 50, 200]), rng.choice([None, 0, 77])), rng.choice([0, 13]))
  elif kind == "chunked":
    mask = mask_lib.ChunkedCausalMask((sq, skv), rng.choice([64, 100, 256]))
  elif kind == "table":
    mask = mask_lib.make_random_mask((sq, skv), rng.choice([0.3, 0.7]), rng.randint(0, 99))
  elif kind == "full":
    mask = mask_lib.FullMask((sq, skv))
  else:
    mask = mask_lib.LocalMask((sq, skv), (150, None), 0) & mask_lib.CausalMask((sq, skv))
  seg = None
  if rng.random() < 0.4 and sq == skv:
    ids = np.zeros((b, sq), np.int32)
    for row in range(b):
      for i, cut in enumerate(sorted(rng.sample(range(1, sq), rng.randint(1, 4)))):
        ids[row, cut:] = i + 1
    seg = (ids, ids)
  cap = rng.choice([None, None, None, 5.0, 20.0])
  repeatable = rng.random() < 0.4
  return dict(b=b, hq=hq, hkv=hkv, sq=sq, skv=skv, d_qk=d_qk, d_v=d_v, kind=kind, mask=mask, seg=seg, cap=cap,
              repeatable=repeatable)


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_cases_match_the_oracle(seed):
  dev = torch.device("cuda:0")
  for case in range(CASES_PER_SEED):
    rng = random.Random(seed * 100003 + case)
    c = _draw(rng)
    mask, seg, cap = c["mask"], c["seg"], c["cap"]
    dense = np.asarray(mask[:, :]) if not isinstance(mask, np.ndarray) else mask
    g = torch.Generator().manual_seed(seed * 1000 + case)
    mk = lambda h, s, d: torch.randn(c["b"], h, s, d, generator=g).to(torch.bfloat16)  # pylint: disable=cell-var-from-loop
    q, k, v = mk(c["hq"], c["sq"], c["d_qk"]), mk(c["hkv"], c["skv"], c["d_qk"]), mk(c["hkv"], c["skv"], c["d_v"])
    do = mk(c["hq"], c["sq"], c["d_v"])
    scale = 1 / math.sqrt(c["d_qk"])
    what = {key: val for key, val in c.items() if key not in ("mask", "seg")} | {"case": case, "segments": seg is not None}
    cfg = dataclasses.replace(splash.SplashConfig.get_default(), attn_logits_soft_cap=cap)
    kernel = splash.make_splash_mha(mask, config=cfg, q_seq_shards=1, save_residuals=True,
                                    repeatable_dq=c["repeatable"])
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    seg_dev = None if seg is None else splash.SegmentIds(*(torch.from_numpy(x).to(dev) for x in seg))
    out, res = kernel(qd, kd, vd, seg_dev, logits_scale=scale)
    out.backward(do.to(dev))
    kernel.check_errors()
    for row in range(c["b"]):
      seg_row = None if seg is None else (seg[0][row], seg[1][row])
      ro, rlse, _ = attention_ref.attention_reference(q[row], k[row], v[row], dense, seg_row, scale=scale,
                                                      attn_logits_soft_cap=cap)
      rdq, rdk, rdv = attention_ref.attention_reference_vjp(do[row], q[row], k[row], v[row], dense, seg_row,
                                                            ro.to(torch.bfloat16), rlse, scale=scale,
                                                            attn_logits_soft_cap=cap)
      # rows with no live key are undefined in the reference: they are left out, and so are the
      # gradients of a batch row that has one (its oracle gradients include those rows)
      live = torch.from_numpy(dense.copy())
      if seg_row is not None:
        live &= torch.from_numpy(seg_row[0][:, None] == seg_row[1][None, :])
      rows = live.any(dim=1)
      o_err = (out[row].float().cpu() - ro).abs() - (1e-2 + 4e-3 * ro.abs())
      assert o_err[:, rows].max().item() <= 0, what
      assert (res["logsumexp"][row].cpu() - rlse)[:, rows].abs().max().item() <= 1e-3, what
      if rows.all():
        assert _rel(qd.grad[row], rdq) <= 1e-2, ("dq", what)
        assert _rel(kd.grad[row], rdk) <= 1e-2, ("dk", what)
        assert _rel(vd.grad[row], rdv) <= 1e-2, ("dv", what)
