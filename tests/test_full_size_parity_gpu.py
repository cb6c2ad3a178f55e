"""The kernels at the full sizes of the benchmark workloads, a slice of each compared with the oracle.

One batch row x one kv-head group is independent of the rest of the problem: its o, logsumexp and
dq (all q heads of the group) and the dk / dv of its kv head depend on nothing else, so the dense
fp32 oracle can check them at a cost of seconds while the kernels run the whole workload.
Tolerances are the ones the task states: o max-abs <= 1e-2, logsumexp <= 1e-3, gradients relative
L2 <= 1e-2.  (Reference kernel tests compare the same quantities against the same oracle function:
splash_attention_kernel_test.py:508-524, :659-666.)

Inputs are generated on the device from fixed seeds (N(0,1) rounded to bf16), the slice is copied to
the host for the oracle.
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
DEV = torch.device("cuda:0")
SCALE = 1 / math.sqrt(D)
O_ATOL, LSE_ATOL, GRAD_REL = 1e-2, 1e-3, 1e-2


def _device_inputs(seed, b, hq, hkv, s):
  out = []
  for i, h in enumerate((hq, hkv, hkv, hq)):
    g = torch.Generator(device=DEV).manual_seed(seed + i)
    out.append(torch.randn(b, h, s, D, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16))
  return out


def _rel(a, ref):
  return ((a.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-20)).item()


def _packed_segments(batch, seq, seed):
  """Documents of length U{512..4096} packed into each row, the last one truncated."""
  rng = np.random.default_rng(seed)
  ids = np.zeros((batch, seq), np.int32)
  for b in range(batch):
    pos = doc = 0
    while pos < seq:
      n = int(rng.integers(512, 4097))
      ids[b, pos:pos + n] = doc
      pos += n
      doc += 1
  return ids


def _check_slice(kernel, dense, q, k, v, do, seg, b, kv_head, repeatable_dq_too=False):
  """Runs fwd + bwd on the whole problem and compares (batch row b, kv head) with the oracle."""
  hq, hkv = q.shape[1], k.shape[1]
  group = hq // hkv
  heads = slice(kv_head * group, (kv_head + 1) * group)
  seg_dev = None if seg is None else splash.SegmentIds(seg, seg)
  forms = [kernel] + ([kernel.with_options(repeatable_dq=not kernel.repeatable_dq)] if repeatable_dq_too else [])
  ref = None
  for kern in forms:
    qd, kd, vd = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out, res = kern(qd, kd, vd, seg_dev, logits_scale=SCALE, save_residuals=True)
    out.backward(do)
    kern.check_errors()
    if ref is None:
      seg_cpu = None if seg is None else (seg[b].cpu(), seg[b].cpu())
      sl = lambda t, hs: t[b:b + 1, hs].cpu()
      ref = attention_ref.fwd_bwd(sl(q, heads), sl(k, slice(kv_head, kv_head + 1)), sl(v, slice(kv_head, kv_head + 1)),
                                  sl(do, heads), dense, None if seg_cpu is None else (seg_cpu[0][None], seg_cpu[1][None]),
                                  scale=SCALE)
    ro, rlse, _, rdq, rdk, rdv = ref
    assert (out[b, heads].float().cpu() - ro[0]).abs().max().item() <= O_ATOL
    assert (res["logsumexp"][b, heads].cpu() - rlse[0]).abs().max().item() <= LSE_ATOL
    assert _rel(qd.grad[b, heads], rdq[0]) <= GRAD_REL
    assert _rel(kd.grad[b, kv_head], rdk[0, 0]) <= GRAD_REL
    assert _rel(vd.grad[b, kv_head], rdv[0, 0]) <= GRAD_REL
    del qd, kd, vd, out, res


def test_llama_shape_causal_full_size_slice():
  """B=4, S=8192, Hq=32, Hkv=8, causal; slice = batch row 3, kv head 5 (q heads 20..23); both
  backward forms."""
  b, hq, hkv, s = 4, 32, 8, 8192
  q, k, v, do = _device_inputs(2000, b, hq, hkv, s)
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  _check_slice(kernel, mask_lib.make_causal_mask((s, s)), q, k, v, do, None, 3, 5, repeatable_dq_too=True)


@pytest.mark.parametrize("composed", [False, True])
def test_packed_window_full_size_slice(composed):
  """B=8, S=16384, H=16, window 4096 to the left + causal, documents of 512..4096 tokens packed per
  row as segment ids.  `composed`: the same mask written as LocalMask(4096, None) & CausalMask,
  which has no mask function and so goes through partial_mask_blocks."""
  b, h, s = 8, 16, 16384
  q, k, v, do = _device_inputs(3000, b, h, h, s)
  seg = torch.from_numpy(_packed_segments(b, s, 3000)).to(DEV)
  if composed:
    mask = mask_lib.LocalMask((s, s), (4096, None), 0) & mask_lib.CausalMask((s, s))
  else:
    mask = mask_lib.LocalMask((s, s), (4096, 0), 0)
  kernel = splash.make_splash_mha(mask, q_seq_shards=1)
  if composed:
    assert kernel.mask_function is None and kernel.fwd_mask_info.partial_mask_blocks is not None
  dense = mask_lib.make_local_attention_mask((s, s), (4096, 0))
  _check_slice(kernel, dense, q, k, v, do, seg, 6, 11)


def test_long_context_causal_row_blocks():
  """B=1, S=131072, Hq=64, Hkv=8, causal, on one GPU.  The first and the last 1024 query rows of one
  q head against a row-block oracle (1024 x 131072 logits): o, logsumexp and dq of those rows."""
  hq, hkv, s, rows = 64, 8, 131072, 1024
  q, k, v, do = _device_inputs(4000, 1, hq, hkv, s)
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  q.requires_grad_(True)
  out, res = kernel(q, k, v, logits_scale=SCALE, save_residuals=True)
  out.backward(do)
  kernel.check_errors()
  head = 43
  kv_head = head // (hq // hkv)
  kc, vc = k[0, kv_head:kv_head + 1].cpu(), v[0, kv_head:kv_head + 1].cpu()
  for r0 in (0, s - rows):
    rs = slice(r0, r0 + rows)
    dense = np.arange(r0, r0 + rows)[:, None] >= np.arange(s)[None, :]
    qc, doc = q.detach()[0, head:head + 1, rs].cpu(), do[0, head:head + 1, rs].cpu()
    ro, rlse, _ = attention_ref.attention_reference(qc, kc, vc, dense, scale=SCALE)
    assert (out[0, head, rs].float().cpu() - ro[0]).abs().max().item() <= O_ATOL
    assert (res["logsumexp"][0, head, rs].cpu() - rlse[0]).abs().max().item() <= LSE_ATOL
    rdq, _, _ = attention_ref.attention_reference_vjp(doc, qc, kc, vc, dense, None, ro.to(torch.bfloat16), rlse,
                                                      scale=SCALE)
    assert _rel(q.grad[0, head, rs], rdq[0]) <= GRAD_REL


@pytest.mark.parametrize("p_format", ["e4m3", "f16"])
def test_fp8_prefill_full_size_last_rows(p_format):
  """B=2, S=32768, Hq=32, Hkv=8, causal, e4m3 inputs with per-128-token scales, forward only.  The
  last 2048 query rows of one kv-head group against the oracle on the dequantised tensors, at the
  bounds tests/test_fp8_gpu.py states for each variant (probabilities in e4m3 / kept 16 bits wide)."""
  b, hq, hkv, s, rows = 2, 32, 8, 32768, 2048
  q, k, v, _ = _device_inputs(5000, b, hq, hkv, s)
  qq, kq, vq = (fp8.quantize_e4m3(t) for t in (q, k, v))
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  o, res = fp8.splash_fwd_fp8(kernel, qq, kq, vq, logits_scale=SCALE, save_residuals=True, p_format=p_format)
  kernel.check_errors()
  bi, kv_head = 1, 6
  group = hq // hkv
  heads = slice(kv_head * group, (kv_head + 1) * group)
  rs = slice(s - rows, s)
  deq = lambda t, hs: fp8.dequantize_e4m3(fp8.Fp8Tensor(t.data[bi:bi + 1, hs], t.scale[bi:bi + 1, hs]), torch.float32)[0].cpu()
  qe, ke, ve = deq(qq, heads)[:, rs], deq(kq, slice(kv_head, kv_head + 1)), deq(vq, slice(kv_head, kv_head + 1))
  dense = np.arange(s - rows, s)[:, None] >= np.arange(s)[None, :]
  ref_exact, lse, mx = attention_ref.attention_reference(qe, ke, ve, dense, scale=SCALE)
  assert (res["logsumexp"][bi, heads, rs].cpu() - lse).abs().max().item() <= 1e-3
  assert (res["max_logits"][bi, heads, rs].cpu() - mx).abs().max().item() <= 1e-3
  if p_format == "f16":
    assert (o[bi, heads, rs].float().cpu() - ref_exact).abs().max().item() <= O_ATOL
    return
  ref, _, _ = attention_ref.attention_reference(*(x.to(torch.bfloat16) for x in (qe, ke, ve)), dense, scale=SCALE)
  err = o[bi, heads, rs].float().cpu() - ref
  assert (err.norm() / ref.norm()).item() <= 3e-2
  assert err.abs().max().item() <= 0.25
