"""Ulysses context parallelism on real GPUs (NCCL): sharded == single-GPU result, bit for bit.

Needs at least two GPUs; skipped otherwise.  Ranks are child processes; each compares its
sequence shard of the output and of dQ / dK / dV with a single-GPU run of the same kernels on the
gathered inputs.  Because every rank computes whole heads with deterministic kernels, equality is
exact.
"""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
D = 128


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _worker(rank, world, port, queue, exchange="nccl", repeatable=True):
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
  dev = torch.device("cuda", rank)
  torch.cuda.set_device(dev)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
  try:
    from tokamax_b200 import splash_attention_kernel as splash
    from tokamax_b200 import splash_attention_mask as mask_lib
    from tokamax_b200 import ulysses

    b, hq, hkv, s = 1, 8, 4, 2048
    g = torch.Generator().manual_seed(7)
    mk = lambda h: torch.randn(b, h, s, D, generator=g).to(torch.bfloat16)
    q, k, v, do = (t.to(dev) for t in (mk(hq), mk(hkv), mk(hkv), mk(hq)))
    # split backward: every gradient repeats bit for bit, so the comparison can be exact; with the
    # fused backward dq is summed in an order that changes from run to run and gets a tolerance
    kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1, repeatable_dq=repeatable)
    same_dq = torch.equal if repeatable else (
        lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item() <= 1e-3)
    scale = 1 / math.sqrt(D)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    full = kernel(qf, kf, vf, logits_scale=scale)
    full.backward(do)
    sl = slice(rank * s // world, (rank + 1) * s // world)
    ql, kl, vl = (t[:, :, sl].clone().requires_grad_(True) for t in (q, k, v))
    cp = ulysses.UlyssesSplashAttention(kernel, exchange=exchange)
    ok = True
    for _ in range(2):  # twice: the peer exchange reuses its buffers
      ql.grad = kl.grad = vl.grad = None
      out = cp(ql, kl, vl, logits_scale=scale)
      out.backward(do[:, :, sl].contiguous())
      torch.cuda.synchronize()
      kernel.check_errors()
      ok = ok and (torch.equal(out, full[:, :, sl]) and same_dq(ql.grad, qf.grad[:, :, sl])
                   and torch.equal(kl.grad, kf.grad[:, :, sl]) and torch.equal(vl.grad, vf.grad[:, :, sl]))
    with torch.no_grad():
      ok = ok and torch.equal(cp(ql, kl, vl, logits_scale=scale), full[:, :, sl])
    queue.put((rank, "ok" if ok else "mismatch"))
  except Exception as e:  # pylint: disable=broad-except
    queue.put((rank, f"{type(e).__name__}: {e}"))
  finally:
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange,repeatable", [("nccl", True), ("peer", True), ("fused", True), ("fused", False)])
def test_ulysses_matches_single_gpu_bitwise(exchange, repeatable):
  """("fused", False): the fused backward, whose kernels store dq / dk / dv straight into the ranks
  that own the rows."""
  world = 2
  ctx = mp.get_context("spawn")
  queue = ctx.Queue()
  port = _free_port()
  procs = [ctx.Process(target=_worker, args=(r, world, port, queue, exchange, repeatable)) for r in range(world)]
  for p in procs:
    p.start()
  results = [queue.get(timeout=300) for _ in range(world)]
  for p in procs:
    p.join(timeout=60)
  assert sorted(results) == [(0, "ok"), (1, "ok")], results
