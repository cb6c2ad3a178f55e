"""GPU parity tests: the CUDA kernels (through the Python API -> C ABI) against the CPU oracle.

Tolerances are the ones the task states: forward output max-abs <= 1e-2, logsumexp <= 1e-3
against the fp32 oracle; dQ / dK / dV relative L2 <= 1e-2.
"""
import dataclasses
import math

import numpy as np
import pytest
import torch

from oracle import attention_ref
from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu

O_ATOL, LSE_ATOL, GRAD_REL = 1e-2, 1e-3, 1e-2
D = 128


def _inputs(seed, b, hq, hkv, sq, skv, mqa=False):
  g = torch.Generator().manual_seed(seed)
  mk = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32).to(torch.bfloat16)
  q, do = mk(b, hq, sq, D), mk(b, hq, sq, D)
  if mqa:
    k, v = mk(b, skv, D), mk(b, skv, D)
  else:
    k, v = mk(b, hkv, skv, D), mk(b, hkv, skv, D)
  return q, k, v, do


def _dense(mask):
  q, kv = mask.shape
  return np.asarray(mask[(slice(0, q), slice(0, kv))]).astype(np.bool_)


def _rel(a, ref):
  return ((a.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-20)).item()


def _run_and_compare(kernel, mask_dense, q, k, v, do, seg=None, scale=1.0 / math.sqrt(D)):
  dev = torch.device("cuda:0")
  qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
  seg_dev = None if seg is None else splash.SegmentIds(seg[0].to(dev), seg[1].to(dev))
  out, res = kernel(qd, kd, vd, seg_dev, logits_scale=scale, save_residuals=True)
  out.backward(do.to(dev))
  kernel.check_errors()
  k4 = k if k.dim() == 4 else k[:, None]
  v4 = v if v.dim() == 4 else v[:, None]
  ro, rlse, rmax, rdq, rdk, rdv = attention_ref.fwd_bwd(q, k4, v4, do, mask_dense, seg, scale=scale)
  assert (out.float().cpu() - ro).abs().max().item() <= O_ATOL
  assert (res["logsumexp"].cpu() - rlse).abs().max().item() <= LSE_ATOL
  assert (res["max_logits"].cpu() - rmax).abs().max().item() <= 1e-3 * max(1.0, rmax.abs().max().item())
  dk, dv = kd.grad, vd.grad
  if k.dim() == 3:
    dk, dv = dk[:, None], dv[:, None]
  assert _rel(qd.grad, rdq) <= GRAD_REL
  assert _rel(dk, rdk) <= GRAD_REL
  assert _rel(dv, rdv) <= GRAD_REL
  # the other backward form (split dq / dkv kernels when the kernel object runs the fused one,
  # and the other way round) on the same forward
  other = kernel.with_options(repeatable_dq=not kernel.repeatable_dq)
  q2, k2, v2 = (t.to(dev).requires_grad_(True) for t in (q, k, v))
  out2, _ = other(q2, k2, v2, seg_dev, logits_scale=scale, save_residuals=True)
  out2.backward(do.to(dev))
  other.check_errors()
  assert torch.equal(out2, out)
  dk2, dv2 = (k2.grad, v2.grad) if k.dim() == 4 else (k2.grad[:, None], v2.grad[:, None])
  assert torch.equal(dk2, dk) and torch.equal(dv2, dv)
  assert _rel(q2.grad, rdq) <= GRAD_REL
  return out, res, qd.grad, dk, dv


def test_library_loaded_and_identifies_itself():
  assert b"sm_100a" in _native.lib().splash_version()


def test_c1_causal_mha_1024():
  """The CPU-sized benchmark case: causal, B=2, Hq=Hkv=8, S=1024, D=128."""
  q, k, v, do = _inputs(1000, 2, 8, 8, 1024, 1024)
  mask = mask_lib.CausalMask((1024, 1024))
  kernel = splash.make_splash_mha(mask, q_seq_shards=1)
  _run_and_compare(kernel, _dense(mask), q, k, v, do)


@pytest.mark.parametrize("hq,hkv", [(8, 2), (4, 1), (6, 2)])
def test_gqa_causal(hq, hkv):
  q, k, v, do = _inputs(7, 1, hq, hkv, 512, 512)
  mask = mask_lib.CausalMask((512, 512))
  _run_and_compare(splash.make_splash_mha(mask, q_seq_shards=1), _dense(mask), q, k, v, do)


def test_mqa_unbatched():
  q, k, v, do = _inputs(11, 1, 4, 1, 384, 384, mqa=True)
  mask = mask_lib.CausalMask((384, 384))
  kernel = splash.make_splash_mqa(mask, q_seq_shards=1, save_residuals=True)
  dev = torch.device("cuda:0")
  out, res = kernel(q[0].to(dev), k[0].to(dev), v[0].to(dev), logits_scale=0.1)
  ro, rlse, _ = attention_ref.attention_reference(q[0], k[0], v[0], _dense(mask), scale=0.1)
  assert out.shape == (4, 384, D) and res["logsumexp"].shape == (4, 384)
  assert (out.float().cpu() - ro).abs().max().item() <= O_ATOL
  assert (res["logsumexp"].cpu() - rlse).abs().max().item() <= LSE_ATOL
  q4, k4, v4, do4 = q, k, v, do
  _run_and_compare(splash.make_splash_mqa(mask, q_seq_shards=1), _dense(mask), q4, k4, v4, do4)


MASKS = {
    "full": lambda s: mask_lib.FullMask((s, s)),
    "local_lazy": lambda s: mask_lib.LocalMask((s, s), (200, 72), 0),
    "local_causal_lazy": lambda s: mask_lib.LocalMask((s, s), (300, 0), 0),
    "chunked_lazy": lambda s: mask_lib.ChunkedCausalMask((s, s), 192),
    "causal_offset": lambda s: mask_lib.CausalMask((s, s), 37),
    "and_local_causal": lambda s: mask_lib.LocalMask((s, s), (260, None), 0) & mask_lib.CausalMask((s, s)),
    "or_chunk_local": lambda s: mask_lib.ChunkedCausalMask((s, s), 256) | mask_lib.LocalMask((s, s), (40, 40), 0),
    "random_or_diag": lambda s: mask_lib.NumpyMask(mask_lib.make_random_mask((s, s), 0.7, 5))
    | mask_lib.LocalMask((s, s), (0, 0), 0),
    "numpy_causal": lambda s: mask_lib.NumpyMask(mask_lib.make_causal_mask((s, s))),
}


@pytest.mark.parametrize("name", sorted(MASKS))
def test_mask_kinds(name):
  s = 768
  q, k, v, do = _inputs(3, 1, 4, 2, s, s)
  mask = MASKS[name](s)
  _run_and_compare(splash.make_splash_mha(mask, q_seq_shards=1), _dense(mask), q, k, v, do)


def test_rectangular_cross_attention():
  q, k, v, do = _inputs(5, 2, 2, 2, 256, 640)
  mask = mask_lib.CausalMask((256, 640), offset=384)
  _run_and_compare(splash.make_splash_mha(mask, q_seq_shards=1), _dense(mask), q, k, v, do)


def test_odd_number_of_q_tiles():
  q, k, v, do = _inputs(6, 1, 2, 1, 384, 384)
  mask = mask_lib.CausalMask((384, 384))
  _run_and_compare(splash.make_splash_mha(mask, q_seq_shards=1), _dense(mask), q, k, v, do)


def _packed_segments(batch, s, seed, lo, hi):
  rng = np.random.default_rng(seed)
  ids = np.zeros((batch, s), np.int32)
  for b in range(batch):
    pos, doc = 0, 0
    while pos < s:
      n = int(rng.integers(lo, hi + 1))
      ids[b, pos:pos + n] = doc
      pos += n
      doc += 1
  return torch.from_numpy(ids)


def test_segment_ids_with_local_window():
  """The packed-sequence benchmark case scaled down: window + causal composed with packed documents."""
  s = 1024
  q, k, v, do = _inputs(3000, 2, 4, 4, s, s)
  mask = mask_lib.LocalMask((s, s), (256, 0), 0)
  seg = _packed_segments(2, s, 1, 32, 256)
  _run_and_compare(splash.make_splash_mha(mask, q_seq_shards=1), _dense(mask), q, k, v, do, seg=(seg, seg))


def test_segment_ids_unbatched_vector():
  s = 512
  q, k, v, do = _inputs(9, 1, 2, 2, s, s)
  mask = mask_lib.CausalMask((s, s))
  seg = _packed_segments(1, s, 2, 64, 200)
  kernel = splash.make_splash_mha(mask, q_seq_shards=1, save_residuals=True)
  dev = torch.device("cuda:0")
  out, _ = kernel(q[0].to(dev), k[0].to(dev), v[0].to(dev), splash.SegmentIds(seg[0].to(dev), seg[0].to(dev)),
                  logits_scale=0.0884)
  ro, _, _ = attention_ref.attention_reference(q[0], k[0], v[0], _dense(mask), (seg[0], seg[0]), scale=0.0884)
  assert (out.float().cpu() - ro).abs().max().item() <= O_ATOL


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_segment_aware_schedule_matches_brute_force(kind):
  """splash_segment_schedule keeps exactly the tiles whose segment-id ranges overlap."""
  dev = torch.device("cuda:0")
  s, batch = 1536, 3
  mask = mask_lib.CausalMask((s, s))
  kernel = splash.make_splash_mha(mask, q_seq_shards=1)
  tables = kernel._tables(dev)  # pylint: disable=protected-access
  sched = (tables.fwd, tables.dq, tables.dkv)[kind]
  seg = _packed_segments(batch, s, 5, 100, 700)
  seg_dev = seg.to(dev)
  out, ws = splash._segment_schedule(sched, kind, seg_dev, seg_dev, s, s)  # pylint: disable=protected-access
  torch.cuda.synchronize()
  nt = s // 128
  n_rows, n_ent = sched.n_rows, sched.n_entries
  row_ptr = next(t for t in tables.keep if t.data_ptr() == sched.row_ptr).cpu().numpy()
  entries = next(t for t in tables.keep if t.data_ptr() == sched.entries).cpu().numpy().reshape(-1, 4)
  import ctypes as C
  nbytes = ws.numel()
  raw = ws.cpu().numpy()
  row_end_off = out.row_end - ws.data_ptr()
  ent_off = out.entries - ws.data_ptr()
  row_end = raw[row_end_off:row_end_off + batch * n_rows * 4].view(np.int32).reshape(batch, n_rows)
  got_entries = raw[ent_off:ent_off + batch * n_ent * 16].view(np.int32).reshape(batch, n_ent, 4)
  tiles = seg.numpy().reshape(batch, nt, 128)
  lo, hi = tiles.min(-1), tiles.max(-1)
  overlap = lambda b, qt, kt: not (hi[b, qt] < lo[b, kt] or lo[b, qt] > hi[b, kt])
  # bits 4 / 5: the sub-tile lies inside one segment (the kernels then skip the id comparison)
  one = lambda b, qt, kt: int(lo[b, qt] == hi[b, qt] == lo[b, kt] == hi[b, kt])
  for b in range(batch):
    for r in range(n_rows):
      want = []
      for e in range(row_ptr[r], row_ptr[r + 1]):
        x, st = int(entries[e, 0]), int(entries[e, 1])
        s0, s1 = st & 3, (st >> 2) & 3
        u0 = u1 = 0
        if kind == 0:
          s0 = s0 if s0 and overlap(b, 2 * r, x) else 0
          s1 = s1 if s1 and 2 * r + 1 < nt and overlap(b, 2 * r + 1, x) else 0
          u0 = one(b, 2 * r, x) if s0 else 0
          u1 = one(b, 2 * r + 1, x) if s1 else 0
        elif kind == 1:
          s0, s1 = (s0 if s0 and overlap(b, r, x) else 0), 0
          u0 = one(b, r, x) if s0 else 0
        else:
          s0, s1 = (s0 if s0 and overlap(b, x, r) else 0), 0
          u0 = one(b, x, r) if s0 else 0
        if s0 or s1:
          want.append((x, s0 | (s1 << 2) | (u0 << 4) | (u1 << 5)))
      got = [(int(a[0]), int(a[1])) for a in got_entries[b, row_ptr[r]:row_end[b, r]]]
      assert got == want, (b, r)
  assert out.entries_per_batch == n_ent and (row_end <= row_ptr[1:][None]).all()
  assert (row_end.astype(np.int64) - row_ptr[:-1][None]).sum() < batch * n_ent  # something was dropped
  assert any(int(e[1]) & 0x30 for b in range(batch) for r in range(n_rows)
             for e in got_entries[b, row_ptr[r]:row_end[b, r]])  # and some tiles lie inside one segment


@pytest.mark.parametrize("bq,bkv", [(256, 128), (128, 256), (512, 512)])
def test_block_sizes(bq, bkv):
  s = 1024
  q, k, v, do = _inputs(13, 1, 2, 2, s, s)
  cfg = splash.SplashConfig(block_q=bq, block_kv=bkv, block_q_dkv=bq, block_kv_dkv=bkv)
  for mask in (mask_lib.CausalMask((s, s)),
               mask_lib.LocalMask((s, s), (300, None), 0) & mask_lib.CausalMask((s, s))):
    _run_and_compare(splash.make_splash_mha(mask, config=cfg, q_seq_shards=1), _dense(mask), q, k, v, do)


def test_op_layout_strided_views():
  """[B, T, H, D] storage viewed as [B, H, T, D]: consumed through strides, no copies."""
  b, t, hq, hkv = 2, 512, 4, 2
  g = torch.Generator().manual_seed(21)
  mk = lambda h: torch.randn(b, t, h, D, generator=g).to(torch.bfloat16)
  q_bthd, k_bthd, v_bthd, do_bthd = mk(hq), mk(hkv), mk(hkv), mk(hq)
  mask = mask_lib.CausalMask((t, t))
  kernel = splash.make_splash_mha(mask, q_seq_shards=1)
  perm = lambda x: x.permute(0, 2, 1, 3)
  _run_and_compare(kernel, _dense(mask), perm(q_bthd), perm(k_bthd), perm(v_bthd), perm(do_bthd))
  dev = torch.device("cuda:0")
  qd = q_bthd.to(dev).permute(0, 2, 1, 3)
  assert not qd.is_contiguous()
  out = kernel(qd, k_bthd.to(dev).permute(0, 2, 1, 3), v_bthd.to(dev).permute(0, 2, 1, 3))
  assert out.shape == (b, hq, t, D)


def test_dynamic_mask_kernel():
  s = 512
  q, k, v, do = _inputs(17, 1, 2, 2, s, s)
  dense = mask_lib.make_random_mask((s, s), 0.6, 2) | mask_lib.make_causal_mask((s, s), 0) & \
      mask_lib.make_local_attention_mask((s, s), (0, 0))
  kernel = splash.make_dynamic_splash_mha(torch.from_numpy(dense))
  _run_and_compare(kernel, dense, q, k, v, do)


@pytest.mark.parametrize("repeatable_dq", [True, False])
def test_bitwise_repeatable(repeatable_dq):
  """Split backward: everything repeats bit for bit.  Fused backward (the default): the output,
  dK and dV do (no atomics touch them); dQ is an fp32 sum whose order varies."""
  q, k, v, do = _inputs(23, 1, 8, 2, 1024, 1024)
  mask = mask_lib.CausalMask((1024, 1024))
  kernel = splash.make_splash_mha(mask, q_seq_shards=1, repeatable_dq=repeatable_dq)
  dev = torch.device("cuda:0")
  runs = []
  for _ in range(2):
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    out = kernel(qd, kd, vd, logits_scale=0.0884)
    out.backward(do.to(dev))
    runs.append((out.detach(), qd.grad, kd.grad, vd.grad))
  for i, (a, b) in enumerate(zip(*runs)):
    if i == 1 and not repeatable_dq:
      assert ((a.float() - b.float()).norm() / b.float().norm()).item() <= 1e-3
    else:
      assert torch.equal(a, b)


def test_fused_and_split_backward_agree():
  """dK / dV of the two backward forms come from the same MMAs in the same order: bit-equal.
  dQ differs only by where the fp32 partial sums are rounded."""
  q, k, v, do = _inputs(29, 2, 8, 2, 1024, 1024)
  dev = torch.device("cuda:0")
  grads = []
  for repeatable in (False, True):
    kernel = splash.make_splash_mha(mask_lib.LocalMask((1024, 1024), (300, 0), 0), q_seq_shards=1,
                                    repeatable_dq=repeatable)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    kernel(qd, kd, vd, logits_scale=0.0884).backward(do.to(dev))
    kernel.check_errors()
    grads.append((qd.grad, kd.grad, vd.grad))
  (dq_f, dk_f, dv_f), (dq_s, dk_s, dv_s) = grads
  assert torch.equal(dk_f, dk_s) and torch.equal(dv_f, dv_s)
  assert ((dq_f.float() - dq_s.float()).norm() / dq_s.float().norm()).item() <= 2e-3


def test_full_size_properties_llama_shape():
  """The Llama-3-8B-shape case (B=4, S=8192, Hq=32, Hkv=8) at full size, checked through size-independent identities.

  (1) rows of P sum to one, so with V = 1 the output is exactly 1; (2) the first causal row
  attends to key 0 only; (3) sum_kv dV = sum_q dO over each kv-head group; (4) <q, dq> = <k, dk>
  because both equal sum(dS * S) / scale-free logits.
  """
  dev = torch.device("cuda:0")
  b, hq, hkv, s = 4, 32, 8, 8192
  g = torch.Generator(device=dev).manual_seed(2000)
  mk = lambda h: torch.randn(b, h, s, D, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
  q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  scale = 1 / math.sqrt(D)
  ones = torch.ones_like(v)
  out1 = kernel(q, k, ones, logits_scale=scale)
  assert (out1.float() - 1).abs().max().item() <= 8e-3  # bf16 half-ulp at 1.0 is 3.9e-3
  qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
  out = kernel(qd, kd, vd, logits_scale=scale)
  assert torch.equal(out[:, :, 0], v.repeat_interleave(hq // hkv, 1)[:, :, 0])
  out.backward(do)
  kernel.check_errors()
  group = hq // hkv
  lhs = vd.grad.float().sum(2)
  rhs = do.float().view(b, hkv, group, s, D).sum((2, 3))
  assert ((lhs - rhs).norm() / rhs.norm()).item() <= 5e-3
  qdq = (qd.grad.float() * q.float()).view(b, hkv, group, s, D).sum((2, 3, 4))
  kdk = (kd.grad.float() * k.float()).sum((2, 3))
  # both sides are sums of ~1e8 signed terms; compare as vectors over (batch, kv head)
  assert ((qdq - kdk).norm() / kdk.norm()).item() <= 1e-2


def test_unsupported_and_invalid_arguments():
  dev = torch.device("cuda:0")
  s = 256
  mask = mask_lib.CausalMask((s, s))
  kernel = splash.make_splash_mha(mask, q_seq_shards=1)
  q = torch.zeros(2, s, D, dtype=torch.bfloat16, device=dev)
  with pytest.raises(NotImplementedError):
    kernel(q.float(), q.float(), q.float())
  wide = torch.zeros(2, s, 320, dtype=torch.bfloat16, device=dev)
  with pytest.raises(NotImplementedError):
    kernel(wide, wide, wide)
  with pytest.raises(ValueError):
    kernel(q[:, :128], q, q)
  with pytest.raises(RuntimeError):
    kernel(q.cpu(), q.cpu(), q.cpu())
  with pytest.raises(NotImplementedError):
    splash.make_splash_mha(mask_lib.CausalMask((64, 64)), q_seq_shards=1,
                           config=splash.SplashConfig(block_q=16, block_kv=16))(
                               q[:, :64], q[:, :64], q[:, :64])


@pytest.mark.parametrize("d_qk,d_v", [(64, 64), (96, 128), (128, 32), (40, 72)])
def test_head_dims_below_128_are_read_in_place(d_qk, d_v):
  """Reference head-dim cases (splash_attention_kernel_test.py:233-237) that fit one MMA tile: no
  padded copies, the TMA boxes zero-fill past the end of a row."""
  b, hq, hkv, s = 1, 4, 2, 384
  g = torch.Generator().manual_seed(d_qk + d_v)
  mk = lambda h, d: torch.randn(b, h, s, d, generator=g).to(torch.bfloat16)
  q, k, v, do = mk(hq, d_qk), mk(hkv, d_qk), mk(hkv, d_v), mk(hq, d_v)
  mask = mask_lib.CausalMask((s, s))
  kernel = splash.make_splash_mha(mask, q_seq_shards=1, save_residuals=True)
  dev = torch.device("cuda:0")
  qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
  scale = 1 / math.sqrt(d_qk)
  out, res = kernel(qd, kd, vd, logits_scale=scale)
  assert out.shape == (b, hq, s, d_v)
  out.backward(do.to(dev))
  kernel.check_errors()
  ro, rlse, _, rdq, rdk, rdv = attention_ref.fwd_bwd(q, k, v, do, _dense(mask), None, scale=scale)
  assert ((out.float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (res["logsumexp"].cpu() - rlse).abs().max().item() <= LSE_ATOL
  assert qd.grad.shape == q.shape and kd.grad.shape == k.shape and vd.grad.shape == v.shape
  assert _rel(qd.grad, rdq) <= GRAD_REL and _rel(kd.grad, rdk) <= GRAD_REL and _rel(vd.grad, rdv) <= GRAD_REL


@pytest.mark.parametrize("d_qk,d_v", [(192, 128), (256, 256), (128, 256), (136, 200)])
@pytest.mark.parametrize("kind", ["causal", "local_segments", "table"])
def test_head_dims_above_128(d_qk, d_v, kind):
  """The reference's (192, 128) and (256, 256) head dims (splash_attention_kernel_test.py:233-237)
  and two ragged ones, with grouped q heads: output, logsumexp, max_logits and the three gradients
  against the oracle."""
  b, hq, hkv, s = 2, 4, 2, 640  # five q tiles: the last schedule row of the forward holds one tile only
  g = torch.Generator().manual_seed(d_qk * 3 + d_v)
  mk = lambda h, d: torch.randn(b, h, s, d, generator=g).to(torch.bfloat16)
  q, k, v, do = mk(hq, d_qk), mk(hkv, d_qk), mk(hkv, d_v), mk(hq, d_v)
  seg = None
  if kind == "causal":
    mask = mask_lib.CausalMask((s, s))
  elif kind == "local_segments":
    mask = mask_lib.LocalMask((s, s), (200, 50), 0)
    ids = np.zeros((b, s), np.int32)
    ids[0, 300:] = 1
    ids[1, 100:450] = 1
    ids[1, 450:] = 2
    seg = (ids, ids)
  else:
    mask = mask_lib.make_random_mask((s, s), 0.6, 11) | np.eye(s, dtype=np.bool_)
  kernel = splash.make_splash_mha(mask, q_seq_shards=1, save_residuals=True)
  dev = torch.device("cuda:0")
  qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
  scale = 1 / math.sqrt(d_qk)
  seg_dev = None if seg is None else splash.SegmentIds(*(torch.from_numpy(x).to(dev) for x in seg))
  out, res = kernel(qd, kd, vd, seg_dev, logits_scale=scale)
  out.backward(do.to(dev))
  kernel.check_errors()
  assert out.shape == (b, hq, s, d_v)
  ro, rlse, rmax, rdq, rdk, rdv = attention_ref.fwd_bwd(q, k, v, do, _dense(mask), seg, scale=scale)
  assert ((out.float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (res["logsumexp"].cpu() - rlse).abs().max().item() <= LSE_ATOL
  assert (res["max_logits"].cpu() - rmax).abs().max().item() <= LSE_ATOL
  assert qd.grad.shape == q.shape and kd.grad.shape == k.shape and vd.grad.shape == v.shape
  assert _rel(vd.grad, rdv) <= GRAD_REL, ("dv", _rel(vd.grad, rdv))
  assert _rel(qd.grad, rdq) <= GRAD_REL, ("dq", _rel(qd.grad, rdq))
  assert _rel(kd.grad, rdk) <= GRAD_REL, ("dk", _rel(kd.grad, rdk))


def test_head_dims_above_128_sinks_and_repeatability():
  """Forward with sinks at (256, 256), and the backward twice: bit-identical gradients."""
  b, hq, hkv, s, d = 1, 4, 2, 384, 256
  g = torch.Generator().manual_seed(5)
  mk = lambda h: torch.randn(b, h, s, d, generator=g).to(torch.bfloat16)
  q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
  sinks = torch.tensor([0.3, -0.7, 1.5, 0.0])
  mask = mask_lib.CausalMask((s, s))
  kernel = splash.make_splash_mha(mask, q_seq_shards=1, save_residuals=True)
  dev = torch.device("cuda:0")
  scale = 1 / math.sqrt(d)
  grads = []
  for _ in range(2):
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    out, res = kernel(qd, kd, vd, None, sinks.to(dev), logits_scale=scale)
    out.backward(do.to(dev))
    grads.append((qd.grad.clone(), kd.grad.clone(), vd.grad.clone()))
  kernel.check_errors()
  ro, rlse, rmax = attention_ref.attention_reference(q[0], k[0], v[0], _dense(mask), None, scale=scale, sinks=sinks)
  assert ((out[0].float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (res["logsumexp"][0].cpu() - rlse).abs().max().item() <= LSE_ATOL
  assert (res["max_logits"][0].cpu() - rmax).abs().max().item() <= LSE_ATOL
  for a, c in zip(*grads):
    assert torch.equal(a, c)


def test_small_head_dim_outputs_stay_inside_their_columns():
  """Outputs and gradients that are column slices of wider buffers: nothing is written beyond
  column d (the kernels hold 128-wide tiles internally)."""
  import abi_util

  b, hq, hkv, s, d = 1, 2, 1, 256, 64
  dev = torch.device("cuda:0")
  g = torch.Generator().manual_seed(77)
  wide = lambda h: torch.randn(b, h, s, 128, generator=g).to(torch.bfloat16).to(dev)
  qw, kw, vw, dow = wide(hq), wide(hkv), wide(hkv), wide(hq)
  q, k, v, do = (t[..., :d] for t in (qw, kw, vw, dow))  # row stride 128, 64 columns: read in place
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  tables = kernel._tables(dev, b)  # pylint: disable=protected-access
  lib = _native.lib()
  import ctypes as C
  desc = splash._tensor_desc  # pylint: disable=protected-access
  outs = {n: torch.full((b, h, s, 128), 5.0, dtype=torch.bfloat16, device=dev)
          for n, h in (("o", hq), ("dq", hq), ("dk", hkv), ("dv", hkv))}
  lse = torch.empty((b, hq, s), dtype=torch.float32, device=dev)
  stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
  fa = _native.SplashFwdArgs()
  fa.q, fa.k, fa.v, fa.o = desc(q), desc(k), desc(v), desc(outs["o"][..., :d])
  fa.logsumexp, fa.sched, fa.scale, fa.mask_value = lse.data_ptr(), tables.fwd, 0.125, -1e30
  fa.mask_fn = splash._mask_fn_struct(kernel.mask_function_rule)  # pylint: disable=protected-access
  fa.error_record = tables.error_record.data_ptr()
  _native.check(lib.splash_fwd(C.byref(fa), stream), "splash_fwd")
  for fused in (True, False):
    ba = _native.SplashBwdArgs()
    ba.q, ba.k, ba.v, ba.o, ba.d_o = desc(q), desc(k), desc(v), desc(outs["o"][..., :d]), desc(do)
    ba.dq, ba.dk, ba.dv = (desc(outs[n][..., :d]) for n in ("dq", "dk", "dv"))
    ba.logsumexp, ba.sched_dq, ba.sched_dkv, ba.mask_fn, ba.scale = lse.data_ptr(), tables.dq, tables.dkv, fa.mask_fn, 0.125
    ba.error_record = fa.error_record
    ba.flags = _native.BWD_FUSED_DQ if fused else 0
    nbytes = (lib.splash_bwd_fused_workspace_bytes if fused else lib.splash_bwd_workspace_bytes)(b, hq, s)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    ba.workspace, ba.workspace_bytes = ws.data_ptr(), nbytes
    _native.check(lib.splash_bwd(C.byref(ba), stream), "splash_bwd")
    torch.cuda.synchronize()
    kernel.check_errors()
    for name, t in outs.items():
      assert (t[..., d:] == 5.0).all(), name
      assert not (t[..., :d] == 5.0).all(), name
  ro, _, _, rdq, rdk, rdv = attention_ref.fwd_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), _dense(mask_lib.CausalMask((s, s))),
                                                  None, scale=0.125)
  assert ((outs["o"][..., :d].float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert _rel(outs["dq"][..., :d], rdq) <= GRAD_REL and _rel(outs["dk"][..., :d], rdk) <= GRAD_REL
  assert _rel(outs["dv"][..., :d], rdv) <= GRAD_REL


def test_seq_minor_layouts_give_the_head_dim_minor_result():
  b, hq, hkv, s = 1, 4, 2, 256
  q, k, v, do = _inputs(41, b, hq, hkv, s, s)
  mask = mask_lib.CausalMask((s, s))
  dev = torch.device("cuda:0")
  plain = splash.make_splash_mha(mask, q_seq_shards=1)
  cfg = dataclasses.replace(splash.SplashConfig.get_default(), q_layout=splash.QKVLayout.SEQ_MINOR,
                            k_layout=splash.QKVLayout.SEQ_MINOR, v_layout=splash.QKVLayout.SEQ_MINOR)
  minor = splash.make_splash_mha(mask, q_seq_shards=1, config=cfg)
  qa, ka, va = (t.to(dev).requires_grad_(True) for t in (q, k, v))
  ref = plain(qa, ka, va, logits_scale=0.1)
  ref.backward(do.to(dev))
  qb, kb, vb = (t.to(dev).transpose(-1, -2).contiguous().requires_grad_(True) for t in (q, k, v))  # [B, H, D, S]
  out = minor(qb, kb, vb, logits_scale=0.1)
  out.backward(do.to(dev))
  assert torch.equal(out, ref)
  for got, want in ((qb.grad, qa.grad), (kb.grad, ka.grad), (vb.grad, va.grad)):
    assert got.shape == want.transpose(-1, -2).shape and torch.equal(got.transpose(-1, -2), want)


def test_forward_peer_output_rows_land_in_their_owners_buffers():
  """`SplashFwdArgs.o_peer` on one GPU: two local buffers stand in for the receive buffers of two
  ranks.  Every output row must arrive, bit for bit, in the buffer of the rank that owns it, at this
  rank's head block, and nothing else may be touched."""
  import ctypes as C

  b, hq, hkv, s, d, world, rank = 2, 4, 2, 512, 128, 2, 1
  dev = torch.device("cuda:0")
  g = torch.Generator().manual_seed(91)
  mk = lambda h: torch.randn(b, h, s, d, generator=g).to(torch.bfloat16).to(dev)
  q, k, v = mk(hq), mk(hkv), mk(hkv)
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  s_loc, h_all = s // world, hq * world
  # receive buffers [B, all heads, S / world, D] of the two "ranks", with a guard band in front
  guard = 64
  bufs = [torch.full((guard + b * h_all * s_loc * d,), 7.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
  ptrs = torch.tensor([t.data_ptr() for t in bufs], dtype=torch.int64, device=dev)
  po = _native.SplashPeerOutput()
  po.ptrs, po.base_bytes, po.rows_per_peer = ptrs.data_ptr(), guard * 2, s_loc
  po.stride_b, po.stride_h, po.stride_s, po.head0 = h_all * s_loc * d, s_loc * d, d, rank * hq
  _, _, _, o, _, _, _ = splash.splash_forward(kernel, q, k, v, None, None, 0.09, None, None, 0, o_peer=po)
  torch.cuda.synchronize()
  kernel.check_errors()
  plain = kernel(q, k, v, logits_scale=0.09)
  assert torch.equal(o, plain)
  for peer in range(world):
    assert (bufs[peer][:guard] == 7.0).all()
    got = bufs[peer][guard:].view(b, h_all, s_loc, d)
    assert torch.equal(got[:, rank * hq:(rank + 1) * hq], o[:, :, peer * s_loc:(peer + 1) * s_loc])
    other = torch.cat([got[:, :rank * hq], got[:, (rank + 1) * hq:]], dim=1)
    assert (other == 7.0).all()
  # arguments that cannot be right are refused before anything is launched
  po.rows_per_peer = 200
  with pytest.raises(_native.SplashError):
    splash.splash_forward(kernel, q, k, v, None, None, 0.09, None, None, 0, o_peer=po)


def test_backward_peer_outputs_rows_land_in_their_owners_buffers():
  """`SplashBwdArgs.dq_peer / dk_peer / dv_peer` on one GPU, two local buffers per gradient standing
  in for two ranks: every gradient row arrives, bit-equal to the local copy, at this rank's head
  block of the rank that owns it."""
  b, hq, hkv, s, d, world, rank = 1, 4, 2, 512, 128, 2, 0
  dev = torch.device("cuda:0")
  g = torch.Generator().manual_seed(92)
  mk = lambda h: torch.randn(b, h, s, d, generator=g).to(torch.bfloat16).to(dev)
  q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)  # fused backward
  s_loc = s // world
  _, _, _, o, lse, _, _ = splash.splash_forward(kernel, q, k, v, None, None, 0.09, None, None, 0)

  def receive_buffers(heads):
    h_all = heads * world
    bufs = [torch.full((b, h_all, s_loc, d), 7.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    ptrs = torch.tensor([t.data_ptr() for t in bufs], dtype=torch.int64, device=dev)
    po = _native.SplashPeerOutput()
    po.ptrs, po.base_bytes, po.rows_per_peer = ptrs.data_ptr(), 0, s_loc
    po.stride_b, po.stride_h, po.stride_s, po.head0 = h_all * s_loc * d, s_loc * d, d, rank * heads
    return bufs, ptrs, po

  recv = [receive_buffers(h) for h in (hq, hkv, hkv)]
  dq, dk, dv, _ = splash.splash_backward(kernel, q, k, v, o, lse, do, None, None, 0.09, 0,
                                         peers=tuple(po for _, _, po in recv))
  torch.cuda.synchronize()
  kernel.check_errors()
  # every kernel writes its local and its remote copy from the same registers, so the two agree bit for
  # bit — dq too, although the fused backward's dq differs in its last bits from run to run
  for (bufs, _, _), local, heads in zip(recv, (dq, dk, dv), (hq, hkv, hkv)):
    for peer in range(world):
      got = bufs[peer][:, rank * heads:(rank + 1) * heads]
      want = local[:, :, peer * s_loc:(peer + 1) * s_loc]
      assert torch.equal(got, want)
      assert (bufs[peer][:, (rank + 1) * heads:] == 7.0).all()
  # the split backward has no second destination
  split = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1, repeatable_dq=True)
  with pytest.raises(_native.SplashError):
    splash.splash_backward(split, q, k, v, o, lse, do, None, None, 0.09, 0, peers=tuple(po for _, _, po in recv))
