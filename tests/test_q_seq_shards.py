"""Kernels built with q_seq_shards > 1 (reference splash_attention_kernel.py:2023-2053).

CPU: the block grid cut from shard i of the sharded MaskInfo tables equals the grid of the
unsharded tables of rows [i*S/n, (i+1)*S/n) — the sharded tables themselves are pinned bit for bit
against the reference's builder by the golden cases.  Two gloo ranks check the wrapper's only
collective (the K / V gradient sum) with the oracle standing in for the kernel.
GPU: every shard's output, logsumexp and dq equal the corresponding rows of the unsharded kernel;
dk / dv summed over the shards match the oracle.
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
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import splash_attention_mask_info as mi

D = 128


def _masks(s):
  return {
      "causal": mask_lib.CausalMask((s, s)),
      "local": mask_lib.LocalMask((s, s), (200, 60), 0),
      "composed": mask_lib.LocalMask((s, s), (300, None), 0) & mask_lib.CausalMask((s, s)),
      "random": mask_lib.NumpyMask(mask_lib.make_random_mask((s, s), 0.3, 7) | np.eye(s, dtype=np.bool_)),
      "full": mask_lib.FullMask((s, s)),
  }


@pytest.mark.parametrize("name", ["causal", "local", "composed", "random", "full"])
@pytest.mark.parametrize("n_shards", [2, 4])
@pytest.mark.parametrize("is_dkv,dynamic", [(False, True), (True, False), (True, True)])
def test_shard_grids_equal_the_grids_of_the_row_slices(name, n_shards, is_dkv, dynamic):
  s, blk = 1024, 128
  mask = _masks(s)[name]
  dense = np.asarray(mask[:, :])
  info, _ = mi.process_mask(mask, (blk, blk), is_dkv=is_dkv, q_seq_shards=n_shards,
                            **({} if not is_dkv else {"return_dynamic_grid": dynamic}))
  nq, nkv = s // blk // n_shards, s // blk
  for shard in range(n_shards):
    rows = dense[shard * s // n_shards:(shard + 1) * s // n_shards]
    ref_info, _ = mi.process_mask(mask_lib.NumpyMask(rows), (blk, blk), is_dkv=is_dkv,
                                  **({} if not is_dkv else {"return_dynamic_grid": dynamic}))
    want_state, want_pid = mi.block_grids(ref_info, nq, nkv, is_dkv=is_dkv)
    got_state, got_pid = mi.block_grids(info, nq, nkv, is_dkv=is_dkv, shard=shard, n_shards=n_shards)
    np.testing.assert_array_equal(got_state, want_state)
    # partial-block ids differ between the two tables (global dedup vs per-slice); the blocks they name must not
    if info.partial_mask_blocks is not None:
      for qi, ki in zip(*np.nonzero(got_state == 1)):
        a = np.asarray(info.partial_mask_blocks[got_pid[qi, ki]])
        b = np.asarray(ref_info.partial_mask_blocks[want_pid[qi, ki]])
        np.testing.assert_array_equal(a, b)
  with pytest.raises(ValueError):
    mi.block_grids(info, nq, nkv, is_dkv=is_dkv, shard=n_shards, n_shards=n_shards)


def _free_port():
  with socket.socket() as sock:
    sock.bind(("127.0.0.1", 0))
    return sock.getsockname()[1]


def _oracle_attention(dense, n_shards):
  """Stand-in for a sharded kernel object on CPU: differentiable dense attention on shard rows."""
  def attention(q, k, v, segment_ids, *, logits_scale, q_shard):
    rows = dense.shape[0] // n_shards
    m = torch.from_numpy(dense[q_shard * rows:(q_shard + 1) * rows])
    group = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(group, 1).float(), v.repeat_interleave(group, 1).float()
    logits = torch.einsum("bhqd,bhkd->bhqk", q.float(), kk) * logits_scale
    logits = logits.masked_fill(~m, -1e30)
    return torch.einsum("bhqk,bhkd->bhqd", torch.softmax(logits, -1), vv).to(q.dtype)
  attention.q_seq_shards = n_shards
  return attention


def _gloo_worker(rank, world, port, queue):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    from tokamax_b200 import q_seq_sharding

    b, hq, hkv, s = 1, 4, 2, 256
    g = torch.Generator().manual_seed(3)
    mk = lambda h: torch.randn(b, h, s, 32, generator=g)
    q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
    dense = np.asarray(mask_lib.make_causal_mask((s, s)))
    full = _oracle_attention(dense, 1)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    full(qf, kf, vf, None, logits_scale=0.2, q_shard=0).backward(do)
    sl = slice(rank * s // world, (rank + 1) * s // world)
    ql, kl, vl = q[:, :, sl].clone().requires_grad_(True), k.clone().requires_grad_(True), v.clone().requires_grad_(True)
    out = q_seq_sharding.QSeqShardedSplashAttention(_oracle_attention(dense, world))(ql, kl, vl, logits_scale=0.2)
    out.backward(do[:, :, sl])
    close = lambda a, r: torch.allclose(a, r, rtol=1e-4, atol=1e-5)
    ok = close(ql.grad, qf.grad[:, :, sl]) and close(kl.grad, kf.grad) and close(vl.grad, vf.grad)
    try:
      q_seq_sharding.QSeqShardedSplashAttention(_oracle_attention(dense, world + 1))(ql, kl, vl)
      ok = False
    except ValueError:
      pass
    queue.put((rank, "ok" if ok else "mismatch"))
  except Exception as e:  # pylint: disable=broad-except
    queue.put((rank, f"{type(e).__name__}: {e}"))
  finally:
    dist.destroy_process_group()


def test_wrapper_sums_kv_gradients_over_two_gloo_ranks():
  world = 2
  ctx = mp.get_context("spawn")
  queue = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, queue)) for r in range(world)]
  for p in procs:
    p.start()
  results = [queue.get(timeout=120) for _ in range(world)]
  for p in procs:
    p.join(timeout=30)
  assert sorted(results) == [(0, "ok"), (1, "ok")], results


@pytest.mark.gpu
@pytest.mark.parametrize("name,n_shards,with_segments", [("causal", 2, False), ("causal", 4, True), ("local", 2, False),
                                                         ("composed", 4, False), ("random", 2, True)])
def test_sharded_kernel_equals_unsharded_rows(name, n_shards, with_segments):
  from tokamax_b200 import splash_attention_kernel as splash

  dev = torch.device("cuda:0")
  b, hq, hkv, s = 2, 4, 2, 1024
  scale = 1 / math.sqrt(D)
  g = torch.Generator().manual_seed(11)
  mk = lambda h: torch.randn(b, h, s, D, generator=g).to(torch.bfloat16)
  q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
  mask = _masks(s)[name]
  seg = seg_cpu = None
  if with_segments:
    ids = torch.from_numpy(np.repeat(np.arange(4, dtype=np.int32), s // 4))[None].expand(b, -1).contiguous()
    seg_cpu = (ids, ids)
    seg = splash.SegmentIds(ids.to(dev), ids.to(dev))
  whole = splash.make_splash_mha(mask, q_seq_shards=1, save_residuals=True, repeatable_dq=True)
  qw, kw, vw = (t.to(dev).requires_grad_(True) for t in (q, k, v))
  ow, rw = whole(qw, kw, vw, seg, logits_scale=scale)
  ow.backward(do.to(dev))
  whole.check_errors()
  sharded = splash.make_splash_mha(mask, q_seq_shards=n_shards, save_residuals=True, repeatable_dq=True)
  assert sharded.q_seq_shards == n_shards
  counts = sharded.fwd_mask_info.num_active_blocks
  assert counts is None or len(counts) == n_shards
  dk_sum = torch.zeros_like(kw, dtype=torch.float32)
  dv_sum = torch.zeros_like(vw, dtype=torch.float32)
  rows = s // n_shards
  for i in range(n_shards):
    sl = slice(i * rows, (i + 1) * rows)
    qi = q[:, :, sl].to(dev).requires_grad_(True)
    ki, vi = (t.to(dev).requires_grad_(True) for t in (k, v))
    seg_i = None if seg is None else splash.SegmentIds(seg.q[:, sl].contiguous(), seg.kv)
    oi, ri = sharded(qi, ki, vi, seg_i, logits_scale=scale, q_shard=i)
    oi.backward(do[:, :, sl].to(dev))
    sharded.check_errors()
    assert torch.equal(oi, ow[:, :, sl]) and torch.equal(ri["logsumexp"], rw["logsumexp"][:, :, sl])
    assert torch.equal(qi.grad, qw.grad[:, :, sl])
    dk_sum += ki.grad.float()
    dv_sum += vi.grad.float()
  dense = np.asarray(mask[:, :])
  _, _, _, _, rdk, rdv = attention_ref.fwd_bwd(q, k, v, do, dense, seg_cpu, scale=scale)
  rel = lambda a, r: ((a.cpu() - r).norm() / r.norm()).item()
  assert rel(dk_sum, rdk) <= 1e-2 and rel(dv_sum, rdv) <= 1e-2
  with pytest.raises(ValueError):
    sharded(q.to(dev), k.to(dev), v.to(dev), logits_scale=scale)  # all rows at once do not fit a shard
  with pytest.raises(ValueError):
    sharded(q[:, :, :rows].to(dev), k.to(dev), v.to(dev), q_shard=n_shards)
