"""Op-level entry point (dot_product_attention, implementation="cuda_sm100") against the oracle."""
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref
from tokamax_b200 import op
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
D = 128


def _bthd(seed, b, t, n):
  g = torch.Generator().manual_seed(seed)
  return torch.randn(b, t, n, D, generator=g).to(torch.bfloat16)


def _oracle(q, k, v, mask, scale):
  outs = []
  for b in range(q.shape[0]):
    o, _, _ = attention_ref.attention_reference(q[b].permute(1, 0, 2), k[b].permute(1, 0, 2), v[b].permute(1, 0, 2),
                                                mask, scale=scale)
    outs.append(o.permute(1, 0, 2))
  return torch.stack(outs)


@pytest.mark.parametrize("kind", ["causal", "full", "local", "local_causal", "bool_mask"])
def test_op_matches_oracle(kind):
  b, t, n, kh = 2, 384, 4, 2
  q, k, v = _bthd(1, b, t, n), _bthd(2, b, t, kh), _bthd(3, b, t, kh)
  dev = torch.device("cuda:0")
  kwargs, dense = {}, np.ones((t, t), bool)
  if kind == "causal":
    kwargs, dense = dict(is_causal=True), mask_lib.make_causal_mask((t, t))
  elif kind == "local":
    kwargs, dense = dict(local_window_size=(100, 28)), mask_lib.make_local_attention_mask((t, t), (100, 28))
  elif kind == "local_causal":
    kwargs = dict(local_window_size=150, is_causal=True)
    dense = mask_lib.make_local_attention_mask((t, t), (150, 0))
  elif kind == "bool_mask":
    dense = mask_lib.make_random_mask((t, t), 0.5, 4) | np.eye(t, dtype=bool)
    kwargs = dict(mask=torch.from_numpy(dense))
  out = op.dot_product_attention(q.to(dev), k.to(dev), v.to(dev), implementation="cuda_sm100", **kwargs)
  assert out.shape == (b, t, n, D)
  ref = _oracle(q, k, v, dense, 1 / math.sqrt(D))
  # bf16 output: half an ulp is 2^-9 relative, which alone exceeds 1e-2 once |o| >= 4 (rows with
  # few live keys), so the bound is the reference tests' atol + rtol * |ref| form here.
  assert ((out.float().cpu() - ref).abs() <= 1e-2 + 4e-3 * ref.abs()).all()


def _oracle_grads(q, k, v, do, mask, scale):
  """[B, T, N, H] tensors -> oracle (o, dq, dk, dv) in the same layout."""
  hm = lambda x: x.permute(0, 2, 1, 3)
  o, _, _, dq, dk, dv = attention_ref.fwd_bwd(hm(q), hm(k), hm(v), hm(do), mask, scale=scale)
  return tuple(hm(x) for x in (o, dq, dk, dv))


@pytest.mark.parametrize("kind", ["causal", "local", "bool_mask_host", "bool_mask_device", "multi_batch_axes"])
def test_op_gradients_match_oracle(kind):
  """dq / dk / dv through the Op: strided [B, T, N, H] views, in-kernel fp32 scale, GQA head map."""
  dev = torch.device("cuda:0")
  b, t, n, kh = 2, 384, 4, 2
  q, k, v, do = _bthd(11, b, t, n), _bthd(12, b, t, kh), _bthd(13, b, t, kh), _bthd(14, b, t, n)
  kwargs, dense = {}, None
  if kind in ("causal", "multi_batch_axes"):
    kwargs, dense = dict(is_causal=True), mask_lib.make_causal_mask((t, t))
  elif kind == "local":
    kwargs, dense = dict(local_window_size=(100, 28)), mask_lib.make_local_attention_mask((t, t), (100, 28))
  else:
    base = mask_lib.make_random_mask((t, t), 0.5, 4) | np.eye(t, dtype=bool)
    dense = base & mask_lib.make_causal_mask((t, t))
    m = torch.from_numpy(base)
    kwargs = dict(mask=m.to(dev) if kind == "bool_mask_device" else m, is_causal=True)
  scale = 0.11
  ref_o, ref_dq, ref_dk, ref_dv = _oracle_grads(q, k, v, do, dense, scale)
  shape = (lambda x: x.reshape(1, 2, *x.shape[1:])) if kind == "multi_batch_axes" else (lambda x: x)
  qd, kd, vd = (shape(x).to(dev).requires_grad_(True) for x in (q, k, v))
  out = op.dot_product_attention(qd, kd, vd, scale=scale, implementation="cuda_sm100", **kwargs)
  out.backward(shape(do).to(dev))
  rel = lambda a, r: ((a.float().cpu().reshape(r.shape) - r).norm() / r.norm()).item()
  assert ((out.float().cpu().reshape(ref_o.shape) - ref_o).abs() <= 1e-2 + 4e-3 * ref_o.abs()).all()
  assert qd.grad.shape == qd.shape and kd.grad.shape == kd.shape and vd.grad.shape == vd.shape
  assert rel(qd.grad, ref_dq) <= 1e-2 and rel(kd.grad, ref_dk) <= 1e-2 and rel(vd.grad, ref_dv) <= 1e-2


def test_op_backward_and_residuals():
  b, t, n, kh = 1, 256, 2, 1
  dev = torch.device("cuda:0")
  q, k, v = (x.to(dev).requires_grad_(True) for x in (_bthd(4, b, t, n), _bthd(5, b, t, kh), _bthd(6, b, t, kh)))
  out = op.dot_product_attention(q, k, v, is_causal=True, scale=0.1)
  out.float().square().sum().backward()
  assert q.grad.shape == q.shape and k.grad.shape == k.shape and torch.isfinite(v.grad.float()).all()
  o2, (mx, lse) = op.IMPLEMENTATIONS["cuda_sm100"](q.detach(), k.detach(), v.detach(), is_causal=True,
                                                   logits_scale=0.1, return_residuals=True)
  assert mx.shape == (b, n, t) and lse.shape == (b, n, t) and torch.equal(o2, out.detach())


def test_op_dispatch_errors():
  dev = torch.device("cuda:0")
  q = torch.zeros(1, 128, 2, D, dtype=torch.bfloat16, device=dev)
  with pytest.raises(NotImplementedError):
    op.dot_product_attention(q, q, q, bias=torch.zeros(1, device=dev), implementation="cuda_sm100")
  with pytest.raises(ExceptionGroup):
    op.dot_product_attention(q, q, q, query_seq_lengths=torch.tensor([64]),
                             implementation=["cuda_sm100", "cuda_sm100"])
  with pytest.raises(ValueError):
    op.dot_product_attention(q, q, q, implementation="nope")
  with pytest.raises(ValueError):
    op.dot_product_attention(q, q, q, implementation=[])


def test_op_soft_cap_matches_oracle():
  b, t, n, kh = 1, 256, 4, 2
  q, k, v = _bthd(21, b, t, n), _bthd(22, b, t, kh), _bthd(23, b, t, kh)
  dev = torch.device("cuda:0")
  out = op.dot_product_attention(q.to(dev), k.to(dev), v.to(dev), is_causal=True, scale=0.3,
                                 logits_soft_cap=5.0, implementation="cuda_sm100")
  o, _, _ = attention_ref.attention_reference(q[0].permute(1, 0, 2), k[0].permute(1, 0, 2), v[0].permute(1, 0, 2),
                                              mask_lib.make_causal_mask((t, t)), scale=0.3, attn_logits_soft_cap=5.0)
  ref = o.permute(1, 0, 2)[None]
  assert ((out.float().cpu() - ref).abs() <= 1e-2 + 4e-3 * ref.abs()).all()


@pytest.mark.parametrize("d_qk,d_v", [(192, 128), (256, 256), (64, 64)])
def test_op_head_dims_other_than_128(d_qk, d_v):
  """[B, T, N, H] strided views at the reference's other head dims (its kernel test draws (64, 64),
  (192, 128) and (256, 256)): output and the three gradients against the oracle."""
  dev = torch.device("cuda:0")
  b, t, n, kh = 2, 384, 4, 2
  g = torch.Generator().manual_seed(d_qk + d_v)
  mk = lambda heads, d: torch.randn(b, t, heads, d, generator=g).to(torch.bfloat16)
  q, k, v, do = mk(n, d_qk), mk(kh, d_qk), mk(kh, d_v), mk(n, d_v)
  scale = d_qk ** -0.5
  ref_o, ref_dq, ref_dk, ref_dv = _oracle_grads(q, k, v, do, mask_lib.make_causal_mask((t, t)), scale)
  qd, kd, vd = (x.to(dev).requires_grad_(True) for x in (q, k, v))
  out = op.dot_product_attention(qd, kd, vd, is_causal=True, implementation="cuda_sm100")  # AUTO scale = d_qk ** -0.5
  out.backward(do.to(dev))
  assert out.shape == (b, t, n, d_v)
  rel = lambda a, r: ((a.float().cpu() - r).norm() / r.norm()).item()
  assert ((out.float().cpu() - ref_o).abs() <= 1e-2 + 4e-3 * ref_o.abs()).all()
  assert rel(qd.grad, ref_dq) <= 1e-2 and rel(kd.grad, ref_dk) <= 1e-2 and rel(vd.grad, ref_dv) <= 1e-2
