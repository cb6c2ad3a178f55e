"""CPU oracle for splash attention numerics.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import this module; the product (``tokamax_b200``) never does.

A torch-CPU fp32 restatement of the reference's dense attention oracle in
``tokamax/_src/ops/experimental/tpu/splash_attention/base.py``:

  forward   ``_attention_reference_impl``        base.py:74-112
  backward  ``_attention_reference_custom_bwd``  base.py:115-173
  GQA/MQA   ``attention_reference``              base.py:185-229 (kv heads repeated, :217-226)
            ``attention_reference_vjp``          base.py:235-285 (group sum, :268-283)

The reference applies no softmax scale (its callers pre-scale q, see
tokamax/_src/ops/attention/pallas_mosaic_tpu.py:112); here ``scale`` multiplies the fp32
logits, which is the same function of the inputs up to the rounding of ``q * scale``.

Pinning: the reference holds no stored golden tensors for this path (its kernel tests compare
against this very function at run time, splash_attention_kernel_test.py:422,508-524).  The
restatement is pinned against the reference's own functions: ``base.py`` is loaded unmodified
(oracle/ref_loader.py: load_reference_base) with numpy standing in for ``jax.numpy`` — JAX is not
installed where this was built, so the arithmetic is numpy's fp32 rather than XLA's, which changes
the order of summation and nothing else — and the outputs of its ``attention_reference`` (with
residuals) and ``attention_reference_vjp`` (both ``backward_impl`` values; MHA, GQA, MQA, segment
ids, sinks, soft cap, head_dim_v != head_dim) are committed as tests/golden/attention_golden.npz
(generator: tests/golden/gen_attention_golden.py); tests/test_oracle.py compares this module with
them to fp32 noise, and repeats the comparison live on random cases where a checkout of the
reference is at hand.  It is also checked against (1) an independent float64 numpy evaluation and
(2) torch autograd of the forward for the backward formulas.  The MaskInfo half of the path is
pinned against the reference's own code as well (see oracle/ref_loader.py).
"""

from __future__ import annotations

import numpy as np
import torch

DEFAULT_MASK_VALUE = -0.7 * float(np.finfo(np.float32).max)


def _one_head_fwd(q, k, v, mask, seg_q, seg_kv, mask_value, soft_cap, scale, sink=None):
  """base.py:74-112 for one head: q [S,D], k [T,D], v [T,Dv], mask bool [S,T]; sink scalar."""
  logits = (q.float() @ k.float().T) * scale  # base.py:85
  if seg_q is not None:
    mask = mask & (seg_q[:, None] == seg_kv[None, :])  # base.py:87-90
  if soft_cap is not None:
    logits = torch.tanh(logits / soft_cap) * soft_cap  # base.py:92-94
  logits = torch.where(mask, logits, torch.tensor(mask_value, dtype=torch.float32))  # :99
  m = logits.max(dim=-1).values  # :100
  if sink is not None:
    m = torch.maximum(m, sink.float())  # :101-102
  s = torch.exp(logits - m[:, None])  # :103
  l = s.sum(dim=-1)  # :104
  if sink is not None:
    l = l + torch.exp(sink.float() - m)  # :104
  p = s / l[:, None]  # :105
  o = p @ v.float()  # :107
  return o, m + torch.log(l), m  # :110


def attention_reference(q, k, v, mask, segment_ids=None, *, scale=1.0, mask_value=DEFAULT_MASK_VALUE,
                        attn_logits_soft_cap=None, sinks=None):
  """fp32 forward.  q [Hq,S,D], k/v [Hkv,T,D] (or [T,D] for MQA), mask bool [S,T], sinks [Hq].

  Returns ``(o [Hq,S,Dv] fp32, logsumexp [Hq,S], max_logits [Hq,S])``.
  """
  mask = torch.as_tensor(np.asarray(mask), dtype=torch.bool)
  if k.dim() == 2:
    k, v = k[None], v[None]
  hq, hkv = q.shape[0], k.shape[0]
  assert hq % hkv == 0
  group = hq // hkv
  seg_q = seg_kv = None
  if segment_ids is not None:
    seg_q, seg_kv = torch.as_tensor(segment_ids[0]), torch.as_tensor(segment_ids[1])
  outs, lses, maxes = [], [], []
  for h in range(hq):
    o, lse, m = _one_head_fwd(q[h], k[h // group], v[h // group], mask, seg_q, seg_kv, mask_value,
                              attn_logits_soft_cap, scale, None if sinks is None else sinks[h])
    outs.append(o)
    lses.append(lse)
    maxes.append(m)
  return torch.stack(outs), torch.stack(lses), torch.stack(maxes)


def _one_head_bwd(do, q, k, v, mask, seg_q, seg_kv, o, lse, mask_value, soft_cap, scale, backward_impl):
  """base.py:115-173 for one head."""
  raw = (q.float() @ k.float().T) * scale  # :129-131
  logits = torch.tanh(raw / soft_cap) * soft_cap if soft_cap is not None else raw  # :133-137
  if seg_q is not None:
    mask = mask & (seg_q[:, None] == seg_kv[None, :])  # :139-142
  logits = torch.where(mask, logits, torch.tensor(mask_value, dtype=torch.float32))  # :143
  p = torch.exp(logits - lse[:, None])  # :145
  do = do.float()
  dv = p.T @ do  # :147
  dp = do @ v.float().T  # :148
  if backward_impl == "flash":
    di = (o.float() * do).sum(-1, keepdim=True)  # :155
  else:
    di = (dp * p).sum(-1, keepdim=True)  # :157
  ds = (dp - di) * p  # :158
  if soft_cap is not None:  # :159-163
    d = torch.tanh(raw / soft_cap)
    g = ds * (1 - d)
    ds = g + g * d
  dk = (ds.T @ q.float()) * scale  # :164 (scale: d logits / d k = scale * q)
  dq = (ds @ k.float()) * scale  # :165
  return dq, dk, dv


def sinks_vjp(do, o, logsumexp, sinks):
  """base.py:166-172: dsinks[h] = sum over rows and columns of -exp(sink - lse) * o * do."""
  w = -torch.exp(sinks.float()[:, None] - logsumexp.float())  # [Hq, S]
  return (w[..., None] * o.float() * do.float()).sum(dim=(-1, -2))


def attention_reference_vjp(do, q, k, v, mask, segment_ids, o, logsumexp, *, scale=1.0,
                            mask_value=DEFAULT_MASK_VALUE, attn_logits_soft_cap=None,
                            backward_impl="flash"):
  """fp32 backward.  Returns ``(dq [Hq,S,D], dk [Hkv,T,D], dv [Hkv,T,Dv])`` in fp32.

  Sinks change nothing here beyond the logsumexp passed in (base.py:145 uses it as is); their own
  gradient is :func:`sinks_vjp`.
  """
  mask = torch.as_tensor(np.asarray(mask), dtype=torch.bool)
  mqa = k.dim() == 2
  if mqa:
    k, v = k[None], v[None]
  hq, hkv = q.shape[0], k.shape[0]
  group = hq // hkv
  seg_q = seg_kv = None
  if segment_ids is not None:
    seg_q, seg_kv = torch.as_tensor(segment_ids[0]), torch.as_tensor(segment_ids[1])
  dq = []
  dk = torch.zeros(k.shape, dtype=torch.float32)
  dv = torch.zeros(v.shape, dtype=torch.float32)
  for h in range(hq):
    a, b, c = _one_head_bwd(do[h], q[h], k[h // group], v[h // group], mask, seg_q, seg_kv, o[h],
                            logsumexp[h], mask_value, attn_logits_soft_cap, scale, backward_impl)
    dq.append(a)
    dk[h // group] += b  # base.py:276-283
    dv[h // group] += c
  if mqa:
    dk, dv = dk[0], dv[0]
  return torch.stack(dq), dk, dv


def fwd_bwd(q, k, v, do, mask, segment_ids=None, *, scale=1.0):
  """Batched convenience: tensors [B,H,S,D]; segment_ids (q [B,S], kv [B,T]) or None."""
  outs = []
  for b in range(q.shape[0]):
    seg = None if segment_ids is None else (segment_ids[0][b], segment_ids[1][b])
    o, lse, mx = attention_reference(q[b], k[b], v[b], mask, seg, scale=scale)
    # the kernels take di from the stored (rounded) output, as the reference does (kernel :1909)
    o_stored = o.to(q.dtype)
    dq, dk, dv = attention_reference_vjp(do[b], q[b], k[b], v[b], mask, seg, o_stored, lse, scale=scale)
    outs.append((o, lse, mx, dq, dk, dv))
  return tuple(torch.stack([t[i] for t in outs]) for i in range(6))
