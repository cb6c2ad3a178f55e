"""Case list shared by the attention golden-vector generator and tests/test_oracle.py.

Inputs are drawn from a seeded numpy generator, rounded to bf16 (stored exactly as float32) — q is
pre-scaled by head_dim ** -0.5 as the reference's callers do, since its oracle applies no scale.
"""

from __future__ import annotations

import numpy as np


def _case(name, hq, hkv, s, t, d, dv, mask, *, mqa=False, segments=False, sinks=False, soft_cap=None, seed=0):
  return dict(name=name, hq=hq, hkv=hkv, s=s, t=t, d=d, dv=dv, mask=mask, mqa=mqa, segments=segments, sinks=sinks,
              soft_cap=soft_cap, seed=seed)


CASES = [
    _case("mha_causal", 2, 2, 96, 96, 64, 64, "causal", seed=1),
    _case("gqa_local_segments", 4, 2, 96, 96, 32, 32, "local", segments=True, seed=2),
    _case("mqa_random_rect", 3, 1, 64, 96, 128, 128, "random", mqa=True, seed=3),
    _case("gqa_causal_sinks", 4, 2, 64, 64, 64, 64, "causal", sinks=True, seed=4),
    _case("gqa_causal_soft_cap", 4, 2, 96, 96, 32, 32, "causal", soft_cap=5.0, seed=5),
    _case("mha_dv_differs", 2, 2, 64, 64, 64, 32, "causal", seed=6),
    _case("mqa_soft_cap_sinks_segments", 4, 1, 96, 96, 32, 32, "causal", mqa=True, segments=True, sinks=True,
          soft_cap=20.0, seed=7),
]
# cases whose backward is also stored for backward_impl="vanilla" (di from dp * p instead of o * do)
VANILLA_TOO = ("mha_causal", "mqa_soft_cap_sinks_segments")


def to_bf16(x: np.ndarray) -> np.ndarray:
  """Round-to-nearest-even to bfloat16, returned as float32."""
  u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
  rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
  return rounded.astype(np.uint32).view(np.float32)


def build(case):
  """(q, k, v, do, mask, segment ids or None, sinks or None) as numpy arrays."""
  rng = np.random.default_rng(1000 + case["seed"])
  hq, hkv, s, t, d, dv = (case[key] for key in ("hq", "hkv", "s", "t", "d", "dv"))
  q = to_bf16(rng.standard_normal((hq, s, d)) * d ** -0.5)
  kshape, vshape = ((t, d), (t, dv)) if case["mqa"] else ((hkv, t, d), (hkv, t, dv))
  k, v = to_bf16(rng.standard_normal(kshape)), to_bf16(rng.standard_normal(vshape))
  do = to_bf16(rng.standard_normal((hq, s, dv)))
  rows, cols = np.arange(s)[:, None], np.arange(t)[None, :]
  if case["mask"] == "causal":
    mask = rows >= cols
  elif case["mask"] == "local":
    mask = (cols >= rows - 40) & (cols <= rows + 12)
  else:
    mask = rng.random((s, t)) < 0.5
    mask[:, 0] = True  # every row keeps a key
  seg = None
  if case["segments"]:
    cuts_q = np.sort(rng.choice(np.arange(1, s), size=3, replace=False))
    ids = np.searchsorted(cuts_q, np.arange(s), side="right").astype(np.int32)
    seg = (ids, ids.copy()) if s == t else None
  sinks = to_bf16(rng.standard_normal((hq,))) if case["sinks"] else None
  return q, k, v, do, mask, seg, sinks
