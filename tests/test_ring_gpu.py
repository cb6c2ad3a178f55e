"""Ring attention on the CUDA kernels.

One GPU: (a) the ring's building blocks — per-pair sub-mask kernels, logsumexp merge, backward
with the merged output / logsumexp — run over four virtual shards and compared with the oracle on
the unsharded problem; (b) the ring itself on a process group of one rank.
Two GPUs (skipped otherwise): the ring over NCCL against the single-GPU kernels.
"""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_ref
from tokamax_b200 import ring_attention as ring
from tokamax_b200 import splash_attention_mask as mask_lib

pytestmark = pytest.mark.gpu
D = 128
DEV = "cuda:0"
SCALE = 1 / math.sqrt(D)


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _rel(a, ref):
  return ((a.float().cpu() - ref).norm() / ref.norm().clamp_min(1e-20)).item()


def _inputs(seed, b, hq, hkv, s):
  g = torch.Generator().manual_seed(seed)
  mk = lambda h: torch.randn(b, h, s, D, generator=g).to(torch.bfloat16)
  return mk(hq), mk(hkv), mk(hkv), mk(hq)


@pytest.mark.parametrize("kind", ["causal", "local", "numpy"])
def test_virtual_ring_of_four_matches_oracle(kind):
  p, s, b, hq, hkv = 4, 1024, 1, 3, 1
  n = s // p
  if kind == "causal":
    mask = mask_lib.CausalMask((s, s))
  elif kind == "local":
    mask = mask_lib.LocalMask((s, s), (300, 40), 0)
  else:
    mask = mask_lib.NumpyMask(mask_lib.make_random_mask((s, s), 0.6, 5) | np.eye(s, dtype=bool))
  q, k, v, do = _inputs(31, b, hq, hkv, s)
  ro, rlse, _, rdq, rdk, rdv = attention_ref.fwd_bwd(q, k, v, do, np.asarray(mask[:, :]), None, scale=SCALE)
  qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
  sh = lambda t, i: t[:, :, i * n:(i + 1) * n].contiguous()
  pair = {(r, c): ring.SplashShardAttention(ring.shard_mask(mask, r, c, p, p)) for r in range(p) for c in range(p)}
  if kind == "causal":
    assert all(pair[r, c].empty == (c > r) for r in range(p) for c in range(p))
  outs, lses = [], []
  for r in range(p):
    o_acc = torch.zeros(b, hq, n, D, device=DEV)
    lse_acc = torch.full((b, hq, n), -float("inf"), device=DEV)
    for i in range(p):
      c = (r - i) % p
      if not pair[r, c].empty:
        o_i, lse_i = pair[r, c].forward(sh(qd, r), sh(kd, c), sh(vd, c), None, None, SCALE)
        ring.merge_partial(o_acc, lse_acc, o_i, lse_i)
    outs.append(o_acc.to(torch.bfloat16))
    lses.append(lse_acc)
  out, lse = torch.cat(outs, 2), torch.cat(lses, 2)
  assert ((out.float().cpu() - ro).abs() <= 1e-2 + 4e-3 * ro.abs()).all()
  assert (lse.cpu() - rlse).abs().max() <= 1e-3
  dq = torch.zeros(b, hq, s, D, device=DEV)
  dk = torch.zeros(b, hkv, s, D, device=DEV)
  dv = torch.zeros(b, hkv, s, D, device=DEV)
  for r in range(p):
    for c in range(p):
      if pair[r, c].empty:
        continue
      dq_i, dk_i, dv_i = pair[r, c].backward(sh(qd, r), sh(kd, c), sh(vd, c), outs[r], lses[r], sh(dod, r), None, None,
                                             SCALE)
      dq[:, :, r * n:(r + 1) * n] += dq_i.float()
      dk[:, :, c * n:(c + 1) * n] += dk_i.float()
      dv[:, :, c * n:(c + 1) * n] += dv_i.float()
  for attn in pair.values():
    attn.kernel.check_errors()
  assert _rel(dq, rdq) <= 1e-2 and _rel(dk, rdk) <= 1e-2 and _rel(dv, rdv) <= 1e-2


def test_ring_of_one_rank_equals_the_plain_kernel():
  from tokamax_b200 import splash_attention_kernel as splash

  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
  dist.init_process_group("gloo", rank=0, world_size=1)
  try:
    s = 512
    mask = mask_lib.CausalMask((s, s))
    q, k, v, do = (t.to(DEV) for t in _inputs(32, 2, 4, 2, s))
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    out, res = ring.make_ring_attention(mask, save_residuals=True, repeatable_dq=True)(qa, ka, va, logits_scale=SCALE)
    out.backward(do)
    qb, kb, vb = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref, rres = splash.make_splash_mha_single_device(mask, save_residuals=True, repeatable_dq=True)(
        qb, kb, vb, logits_scale=SCALE)
    ref.backward(do)
    assert torch.equal(out, ref) and torch.equal(res["logsumexp"], rres["logsumexp"])
    assert torch.equal(qa.grad, qb.grad) and torch.equal(ka.grad, kb.grad) and torch.equal(va.grad, vb.grad)
    with pytest.raises(NotImplementedError):
      ring.make_ring_attention(mask)(q, k, v, None, torch.zeros(4, device=DEV))
    with pytest.raises(ValueError):
      ring.make_ring_attention(mask)(q[:, :, :256], k, v)
  finally:
    dist.destroy_process_group()


def test_zigzag_ring_of_one_rank_matches_the_plain_kernel():
  """One rank, two chunks: exercises strided q / k / v pieces and the per-chunk merge on the kernels."""
  from tokamax_b200 import splash_attention_kernel as splash

  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
  dist.init_process_group("gloo", rank=0, world_size=1)
  try:
    s = 1024
    mask = mask_lib.CausalMask((s, s))
    q, k, v, do = (t.to(DEV) for t in _inputs(34, 1, 4, 2, s))
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    out, res = ring.make_ring_attention(mask, save_residuals=True, layout="zigzag")(qa, ka, va, logits_scale=SCALE)
    out.backward(do)
    qb, kb, vb = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref, rres = splash.make_splash_mha_single_device(mask, save_residuals=True)(qb, kb, vb, logits_scale=SCALE)
    ref.backward(do)
    rel = lambda a, r: ((a.float() - r.float()).norm() / r.float().norm()).item()
    assert rel(out, ref) <= 5e-3 and (res["logsumexp"] - rres["logsumexp"]).abs().max() <= 1e-3
    assert rel(qa.grad, qb.grad) <= 1e-2 and rel(ka.grad, kb.grad) <= 1e-2 and rel(va.grad, vb.grad) <= 1e-2
  finally:
    dist.destroy_process_group()


def _worker(rank, world, port, queue):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
  dev = torch.device("cuda", rank)
  torch.cuda.set_device(dev)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
  try:
    from tokamax_b200 import splash_attention_kernel as splash

    b, hq, hkv, s = 1, 6, 2, 2048
    q, k, v, do = (t.to(dev) for t in _inputs(33, b, hq, hkv, s))
    mask = mask_lib.CausalMask((s, s))
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    full, fres = splash.make_splash_mha_single_device(mask, save_residuals=True)(qf, kf, vf, logits_scale=SCALE)
    full.backward(do)
    sl = slice(rank * s // world, (rank + 1) * s // world)
    ql, kl, vl = (t[:, :, sl].clone().requires_grad_(True) for t in (q, k, v))
    out, res = ring.make_ring_attention(mask, save_residuals=True)(ql, kl, vl, logits_scale=SCALE)
    out.backward(do[:, :, sl].contiguous())
    torch.cuda.synchronize()
    rel = lambda a, ref: ((a.float() - ref.float()).norm() / ref.float().norm()).item()
    worst = max(rel(out, full[:, :, sl]), rel(ql.grad, qf.grad[:, :, sl]), rel(kl.grad, kf.grad[:, :, sl]),
                rel(vl.grad, vf.grad[:, :, sl]))
    lse_err = (res["logsumexp"] - fres["logsumexp"][:, :, sl]).abs().max().item()
    queue.put((rank, "ok" if worst <= 1e-2 and lse_err <= 1e-3 else f"mismatch {worst} {lse_err}"))
  except Exception as e:  # pylint: disable=broad-except
    queue.put((rank, f"{type(e).__name__}: {e}"))
  finally:
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ring_matches_single_gpu_on_two_gpus():
  world = 2
  ctx = mp.get_context("spawn")
  queue = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, queue)) for r in range(world)]
  for p in procs:
    p.start()
  results = [queue.get(timeout=300) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
  assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_fused_merge_matches_the_torch_formula():
  g = torch.Generator().manual_seed(9)
  b, h, s = 2, 3, 200
  o_acc = torch.randn(b, h, s, D, generator=g)
  lse_acc = torch.randn(b, h, s, generator=g) * 3
  o_i = torch.randn(b, h, s, D, generator=g).to(torch.bfloat16)
  lse_i = torch.randn(b, h, s, generator=g) * 3
  lse_acc[0, 0, :5] = -float("inf")      # nothing merged yet
  lse_i[0, 1, :5] = -2.0e38              # no live key on this shard
  lse_acc[1, 2, :3] = -2.0e38
  lse_i[1, 2, :3] = -2.0e38              # dead on both
  want_o, want_l = o_acc.clone(), lse_acc.clone()
  ring.merge_partial(want_o, want_l, o_i, lse_i)  # host tensors: the torch form
  got_o, got_l = o_acc.to(DEV), lse_acc.to(DEV)
  ring.merge_partial(got_o, got_l, o_i.to(DEV), lse_i.to(DEV))
  torch.testing.assert_close(got_o.cpu(), want_o, rtol=2e-5, atol=2e-5)
  finite = torch.isfinite(want_l)
  torch.testing.assert_close(got_l.cpu()[finite], want_l[finite], rtol=2e-6, atol=2e-5)
  assert torch.equal(got_o.cpu()[0, 0, :5], o_i[0, 0, :5].float())
  with pytest.raises(ValueError):
    ring.merge_partial(got_o, got_l, o_i.float().to(DEV), lse_i.to(DEV))
