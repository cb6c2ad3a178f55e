#!/usr/bin/env python3
"""Benchmark of the splash-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

A step is one forward + backward of splash attention over one batch of synthetic inputs
(Q, K, V, dO ~ N(0,1) in bf16 from fixed seeds, softmax scale 1/sqrt(128)).  The metric is
mask-counted TFLOP/s: 14 * D * B * Hq * N_live FLOPs per step, N_live = number of unmasked
(query, key) pairs.  Workloads:

  c2  causal, B=4, S=8192, Hq=32, Hkv=8, D=128 (Llama-3-8B shape)        -- default at N=1
  c4  causal, B=1, S=131072, Hq=64, Hkv=8, D=128, Ulysses context parallel -- default at N>1
  c1  causal, B=2, S=1024, Hq=Hkv=8                                        -- the CPU-sized case
  c3  local window 4096 + causal with packed-document segment ids, B=8, S=16384, Hq=Hkv=16

  c5  causal, B=2, S=32768, Hq=32, Hkv=8, e4m3 inputs with per-128-token scales, forward only

One JSON line is printed by rank 0.  At N = 1 the line also carries short runs of c3 and c5 under
``other_workloads``; at N > 1 it carries the same step timed on one GPU alone (``cp.single_gpu_ms_per_step``)
so that the scaling efficiency refers to one workload.  ``--impl reference`` times the CPU restatement
of the reference's own fp32 attention (oracle/) on all host cores on a bounded sample of the same
workload (the reference itself needs JAX, which is not installed here).
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D = 128
SCALE = 1.0 / math.sqrt(D)

WORKLOADS = {
    "c1": dict(config_id=1, batch=2, q_heads=8, kv_heads=8, seq=1024, mask="causal"),
    "c2": dict(config_id=2, batch=4, q_heads=32, kv_heads=8, seq=8192, mask="causal"),
    "c3": dict(config_id=3, batch=8, q_heads=16, kv_heads=16, seq=16384, mask="local4096_causal_segments"),
    "c4": dict(config_id=4, batch=1, q_heads=64, kv_heads=8, seq=131072, mask="causal"),
    "c5": dict(config_id=5, batch=2, q_heads=32, kv_heads=8, seq=32768, mask="causal"),  # e4m3, forward only
}


# ----------------------------------------------------------------------------------------------
# workload construction
# ----------------------------------------------------------------------------------------------
def packed_segments(batch: int, seq: int, seed: int) -> np.ndarray:
  """Documents of length U{512..4096} packed into each row (last one truncated)."""
  rng = np.random.default_rng(seed)
  ids = np.zeros((batch, seq), np.int32)
  for b in range(batch):
    pos, doc = 0, 0
    while pos < seq:
      n = int(rng.integers(512, 4097))
      ids[b, pos:pos + n] = doc
      pos += n
      doc += 1
  return ids


def live_pairs(w: dict, segments: np.ndarray | None) -> int:
  """Unmasked (q, k) pairs summed over the batch (per q head)."""
  s = w["seq"]
  if w["mask"] == "causal":
    return w["batch"] * (s * (s + 1) // 2)
  # window 4096 + causal and documents <= 4096 long: the window never cuts inside a document,
  # so a row keeps exactly its causal prefix within its own document.
  total = 0
  for b in range(w["batch"]):
    _, counts = np.unique(segments[b], return_counts=True)
    total += int(sum(int(c) * (int(c) + 1) // 2 for c in counts))
  return total


def host_inputs(w: dict, heads_q=None, heads_kv=None, batch=None, pin=False):
  cid = w["config_id"]
  b = batch or w["batch"]
  hq, hkv, s = heads_q or w["q_heads"], heads_kv or w["kv_heads"], w["seq"]

  def gen(seed, h):
    g = torch.Generator(device="cpu").manual_seed(seed)
    t = torch.randn(b, h, s, D, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return t.pin_memory() if pin else t

  return gen(1000 * cid + 0, hq), gen(1000 * cid + 1, hkv), gen(1000 * cid + 2, hkv), gen(1000 * cid + 3, hq)


def device_inputs(w: dict, device, heads_q=None, heads_kv=None, seq_slice=None):
  """Same distribution generated on the device (the large configs would take minutes on CPU)."""
  cid = w["config_id"]
  hq, hkv, s = heads_q or w["q_heads"], heads_kv or w["kv_heads"], w["seq"]
  s_loc = s if seq_slice is None else seq_slice
  out = []
  for i, h in enumerate((hq, hkv, hkv, hq)):
    g = torch.Generator(device=device).manual_seed(1000 * cid + i + 17 * (device.index or 0))
    out.append(torch.randn(w["batch"], h, s_loc, D, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16))
  return out


def l2_note(w: dict) -> str:
  """Says whether a step's inputs exceed the 126 MB L2 (the timing rule: larger inputs, or a flush)."""
  mb = 2 * (2 * w["q_heads"] + 2 * w["kv_heads"]) * w["batch"] * w["seq"] * D / 1e6  # q, do, k, v in bf16
  if mb > 126:
    return f"inputs of a step ({mb:.0f} MB of q, k, v, do) are larger than the 126 MB L2; no flush needed"
  return (f"inputs of a step are {mb:.0f} MB and fit the 126 MB L2: this workload is a parity-size case, its "
          "number is launch-bound and is not a bench line")


def make_kernel(w: dict, bwd: str = "fused"):
  from tokamax_b200 import splash_attention_kernel as splash
  from tokamax_b200 import splash_attention_mask as mask_lib

  s = w["seq"]
  if w["mask"] == "causal":
    mask = mask_lib.CausalMask((s, s))
  else:
    mask = mask_lib.LocalMask((s, s), (4096, 0), 0)
  return splash.make_splash_mha(mask, q_seq_shards=1, repeatable_dq=(bwd == "split"))


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
  """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

  FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
            "clocks_event_reasons.sw_power_cap,clocks.mem,clocks.max.mem")

  def __init__(self, index: int):
    self.index = index
    self.rows: list[list[str]] = []
    self.proc = None
    self.thread = None

  def start(self):
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
           "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      self.proc = None
      return
    def pump():
      for line in self.proc.stdout:
        self.rows.append([time.time()] + [c.strip() for c in line.split(",")])
    self.thread = threading.Thread(target=pump, daemon=True)
    self.thread.start()

  def mark(self):
    """Call when the timed region starts: only samples that arrive after this are reported (the
    sampler is started before the warm-up, because nvidia-smi can take longer to produce its first
    line than a short timed region lasts)."""
    self.t0 = time.time()

  def stop(self) -> dict:
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
    if self.thread:
      self.thread.join(timeout=2)
    sm, smax, mem, mem_max, power, reasons = [], [], [], [], [], set()
    names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
    t0 = getattr(self, "t0", 0.0)
    for r in self.rows:
      if r[0] < t0:
        continue
      r = r[1:]
      if len(r) < 7:
        continue
      try:
        sm.append(float(r[0]))
        smax.append(float(r[1]))
      except ValueError:
        continue
      try:
        power.append(float(r[2]))
        mem.append(float(r[7]))
        mem_max.append(float(r[8]))
      except (ValueError, IndexError):
        pass
      for name, val in zip(names, r[3:7]):
        if val.lower().startswith("active"):
          reasons.add(name)
    return {
        "sm_mhz": float(np.median(sm)) if sm else None,
        "sm_max_mhz": float(max(smax)) if smax else None,
        "mem_mhz": float(np.median(mem)) if mem else None,
        "mem_max_mhz": float(max(mem_max)) if mem_max else None,
        "power_w": float(np.median(power)) if power else None,
        "samples": len(sm),
        "reasons": sorted(reasons),
    }


# ----------------------------------------------------------------------------------------------
# timing helpers
# ----------------------------------------------------------------------------------------------
def timed_steps(step_fn, steps: int, warmup: int, barrier=None) -> float:
  """ms per step: warm-up, then `steps` steps between two events on the current stream."""
  for _ in range(warmup):
    step_fn()
  if barrier:
    barrier()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(steps):
    step_fn()
  e1.record()
  torch.cuda.synchronize()
  if barrier:
    barrier()
  return e0.elapsed_time(e1) / steps


def pinned_copy_gbs(device, nbytes: int = 256 << 20) -> dict:
  """Standalone host<->device copy rates of the machine from pinned memory (GB/s), for reading `e2e`:
  a slow end-to-end number on a fast kernel is the host link, not the pipeline."""
  host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
  dev_buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
  out = {}
  for name, fn in (("h2d", lambda: dev_buf.copy_(host, non_blocking=True)),
                   ("d2h", lambda: host.copy_(dev_buf, non_blocking=True))):
    out[name + "_gbs"] = nbytes / timed_steps(fn, 5, 2) / 1e6
  return out


def fp8_gemm_peak_tflops(device) -> float | None:
  """Dense e4m3 x e4m3 -> bf16 GEMM rate of this GPU (torch._scaled_mm, 8192^3, best of 10), the
  denominator for the e4m3 forward; None if the call is not available."""
  try:
    n = 8192
    a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()  # column-major operand
    one = torch.ones((), device=device, dtype=torch.float32)
    fn = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # pylint: disable=protected-access
    fn()
    best = min(timed_steps(fn, 1, 1) for _ in range(10))
    return 2 * n ** 3 / best / 1e9
  except Exception:  # pylint: disable=broad-except
    return None


def measured_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      p = json.load(f)
    return float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
  return 1590.0, 1400.0, "fallback"


# DRAM traffic of one launch of the dominant kernel on the c2 workload (dram__bytes_read.sum +
# dram__bytes_write.sum from an ncu capture of that kernel), per backward form; None: not captured.
KERNEL_TRAFFIC_BYTES_C2 = {"dkv": 841.6e6, "bwd_fused": 1852.0e6}


def per_kernel_times(kernel, q, k, v, do, seg, iters: int = 5) -> dict:
  """Average device time of each kernel of one step, timed alone through the C ABI."""
  from tokamax_b200 import _native
  from tokamax_b200 import splash_attention_kernel as splash

  lib = _native.lib()
  dev = q.device
  tables = kernel._tables(dev)  # pylint: disable=protected-access
  b, hq, s, _ = q.shape
  o = torch.empty_like(q)
  lse = torch.empty((b, hq, s), dtype=torch.float32, device=dev)
  dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
  fa = _native.SplashFwdArgs()
  fa.q, fa.k, fa.v, fa.o = map(splash._tensor_desc, (q, k, v, o))  # pylint: disable=protected-access
  fa.logsumexp = lse.data_ptr()
  fa.q_segment_ids = seg[0].data_ptr() if seg else None
  fa.kv_segment_ids = seg[1].data_ptr() if seg else None
  fwd_sched, dq_sched, dkv_sched, keep = tables.fwd, tables.dq, tables.dkv, []
  if seg:
    for kind, name in ((0, 'fwd'), (1, 'dq'), (2, 'dkv')):
      sc, ws_ = splash._segment_schedule(getattr(tables, name), kind, seg[0], seg[1], s, k.shape[2])  # pylint: disable=protected-access
      keep.append(ws_)
      if kind == 0:
        fwd_sched = sc
      elif kind == 1:
        dq_sched = sc
      else:
        dkv_sched = sc
  fa.sched = fwd_sched
  fa.mask_fn = splash._mask_fn_struct(kernel.mask_function_rule)  # pylint: disable=protected-access
  fa.scale = SCALE
  fa.mask_value = -1e30
  fa.error_record = tables.error_record.data_ptr()
  fused = not kernel.repeatable_dq
  ws_bytes = (lib.splash_bwd_fused_workspace_bytes if fused else lib.splash_bwd_workspace_bytes)(b, hq, s)
  ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
  ba = _native.SplashBwdArgs()
  ba.flags = _native.BWD_FUSED_DQ if fused else 0
  ba.q, ba.k, ba.v, ba.o, ba.d_o = map(splash._tensor_desc, (q, k, v, o, do))  # pylint: disable=protected-access
  ba.dq, ba.dk, ba.dv = map(splash._tensor_desc, (dq, dk, dv))  # pylint: disable=protected-access
  ba.logsumexp = lse.data_ptr()
  ba.q_segment_ids, ba.kv_segment_ids = fa.q_segment_ids, fa.kv_segment_ids
  ba.sched_dq, ba.sched_dkv = dq_sched, dkv_sched
  ba.mask_fn = fa.mask_fn
  ba.scale = SCALE
  ba.workspace, ba.workspace_bytes = ws.data_ptr(), ws_bytes
  ba.error_record = fa.error_record
  stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

  def run_fwd():
    _native.check(lib.splash_fwd(C.byref(fa), stream), "splash_fwd")

  def run_bwd(mask):
    ba.launch_mask = mask
    _native.check(lib.splash_bwd(C.byref(ba), stream), "splash_bwd")

  out = {}
  out["fwd"] = timed_steps(run_fwd, iters, 2)
  run_bwd(1)
  # split form: di pass | dq kernel | dkv kernel.  fused form: di pass + clearing of the fp32 dQ
  # image | cast of the image to bf16 | the fused kernel (dK, dV and the dQ partials)
  out["delta"] = timed_steps(lambda: run_bwd(1), iters, 1)
  out["dq_cast" if fused else "dq"] = timed_steps(lambda: run_bwd(2), iters, 2)
  out["bwd_fused" if fused else "dkv"] = timed_steps(lambda: run_bwd(4), iters, 2)
  kernel.check_errors()
  return out


def _dense_causal(s: int) -> np.ndarray:
  return np.tril(np.ones((s, s), dtype=np.bool_))


def _dense_window_causal(s: int, left: int) -> np.ndarray:
  idx = np.arange(s)
  return (idx[None, :] <= idx[:, None]) & (idx[None, :] >= idx[:, None] - left)


def cpu_baseline(w: dict, seconds_budget: float = 20.0) -> dict:
  """Oracle forward + backward on the host cores over a bounded sample of the workload.

  Touches nothing but the oracle and numpy / torch-CPU (the CUDA library is not loaded here), and
  uses every host core: a launcher may have set OMP_NUM_THREADS=1 for its ranks.
  """
  from oracle import attention_ref

  torch.set_num_threads(os.cpu_count() or 1)
  s = min(w["seq"], 8192)  # the dense fp32 oracle holds S x S logits; cap the sample's sequence
  group = w["q_heads"] // w["kv_heads"]
  g = torch.Generator().manual_seed(1000 * w["config_id"])
  mk = lambda h: torch.randn(1, h, s, D, generator=g, dtype=torch.float32).to(torch.bfloat16)
  q, k, v, do = mk(group), mk(1), mk(1), mk(group)
  if w["mask"] == "causal":
    mask = _dense_causal(s)
    seg = None
    n_live = s * (s + 1) // 2
  else:
    mask = _dense_window_causal(s, 4096)
    ids = packed_segments(1, s, 3)
    seg = (torch.from_numpy(ids), torch.from_numpy(ids))
    n_live = live_pairs(dict(w, batch=1, seq=s), ids)
  flops = 14 * D * group * n_live
  t0 = time.perf_counter()
  reps = 0
  while True:
    attention_ref.fwd_bwd(q, k, v, do, mask, seg, scale=SCALE)
    reps += 1
    dt = time.perf_counter() - t0
    if dt > seconds_budget or reps >= 5:
      break
  return {
      "value": flops * reps / dt / 1e12,
      "unit": "TFLOP/s",
      "cores": torch.get_num_threads(),
      "kind": "port",
      "sample": (f"1 batch row x 1 kv head ({group} q heads) of {w['mask']} seq {s}, fwd+bwd, {reps} reps in "
                 f"{dt:.1f} s; torch-CPU fp32 restatement of the reference's attention_reference[_vjp]"),
      "sample_seq": s,
      "same_seq_as_workload": s == w["seq"],
  }


def maskinfo_build_times(w: dict) -> dict:
  """Host time to build the forward MaskInfo of the workload's mask: the native builder against the
  numpy restatement of the reference's block-by-block `_process_mask` (capped at 16384 tokens for the
  restatement, whose cost grows with the number of blocks times the block area)."""
  from oracle import maskinfo_ref
  from tokamax_b200 import splash_attention_mask as mask_lib
  from tokamax_b200 import splash_attention_mask_info as mask_info_lib

  def build(s):
    return mask_lib.CausalMask((s, s)) if w["mask"] == "causal" else mask_lib.LocalMask((s, s), (4096, 0), 0)

  s = w["seq"]
  mask_info_lib._process_mask.cache_clear()  # pylint: disable=protected-access
  t0 = time.perf_counter()
  mask_info_lib.process_mask(build(s), (128, 128))
  native_ms = (time.perf_counter() - t0) * 1e3
  s_ref = min(s, 16384)
  t0 = time.perf_counter()
  maskinfo_ref.process_mask(build(s_ref), (128, 128), False)
  port_ms = (time.perf_counter() - t0) * 1e3
  return {"native": native_ms, "native_seq": s, "port": port_ms, "port_seq": s_ref}


# ----------------------------------------------------------------------------------------------
# arms
# ----------------------------------------------------------------------------------------------
def run_reference(args, w, wname):
  """CPU arm: the reference's fp32 attention (restated; JAX is absent) on the host cores."""
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return
  for _ in range(min(args.warmup, 1)):
    cpu_baseline(w, seconds_budget=1.0)
  t0 = time.perf_counter()
  vals = [cpu_baseline(w, seconds_budget=4.0) for _ in range(args.steps)]
  dt = (time.perf_counter() - t0) / max(args.steps, 1)
  base = vals[-1]
  value = float(np.mean([v["value"] for v in vals]))
  base["value"] = value
  line = {
      "impl": "reference", "metric": "splash fwd+bwd TFLOP/s (masked FLOPs)", "value": value, "unit": "TFLOP/s",
      "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
      # (as in the product arm: one GPU runs c2 with fixed work per GPU, N > 1 split c4's fixed work)
      "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None,
      "dtype": "f32", "data": "synthetic",
      "config": {"workload": wname, **{k: w[k] for k in ("batch", "q_heads", "kv_heads", "seq", "mask")},
                 "head_dim": D, "sample_seq": base["sample_seq"],
                 "note": "each step is a bounded sample of the workload (one batch row x one kv-head group at "
                         "sample_seq tokens) on all host cores"},
      "cpu_baseline": base,
      "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
      "gpu_launches": 0,
  }
  print(json.dumps(line), flush=True)


def run_single_gpu(args, w, wname, emit=True):
  from tokamax_b200 import splash_attention_kernel as splash

  dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
  torch.cuda.set_device(dev)
  kernel = make_kernel(w, args.bwd)
  seg = seg_np = None
  if "segments" in w["mask"]:
    seg_np = packed_segments(w["batch"], w["seq"], 3000)
    seg_t = torch.from_numpy(seg_np).to(dev)
    seg = (seg_t, seg_t)
  n_live = live_pairs(w, seg_np)
  flops = 14 * D * w["q_heads"] * n_live
  big = w["batch"] * w["q_heads"] * w["seq"] > (1 << 22)
  q, k, v, do = device_inputs(w, dev) if big else [t.to(dev) for t in host_inputs(w)]
  seg_ids = splash.SegmentIds(*seg) if seg else None

  def step():
    qd, kd, vd = q.detach().requires_grad_(True), k.detach().requires_grad_(True), v.detach().requires_grad_(True)
    out = kernel(qd, kd, vd, seg_ids, logits_scale=SCALE)
    out.backward(do)
    return out, qd.grad, kd.grad, vd.grad

  sampler = ClockSampler(dev.index or 0)
  sampler.start()
  for _ in range(args.warmup):
    step()
  torch.cuda.synchronize()
  sampler.mark()
  ms = timed_steps(step, args.steps, 0)
  clocks = sampler.stop()
  kernel.check_errors()
  value = flops / ms / 1e9

  # ---- end to end: host buffers in, host buffers out, through the public API.  Batch rows are
  # independent units of the step.  Copies run on two side streams (pinned memory, full-duplex PCIe)
  # and are double-buffered across steps, the way an input pipeline prefetches: while one unit
  # computes, later units (of this step or the next) come in and earlier results go out; within a
  # unit dO follows q/k/v (the forward does not need it) and the output leaves while the backward
  # runs.  Every step's inputs cross the link and every step's results are back in host memory
  # before the timed region ends.
  e2e = None
  if not args.no_e2e:
    hq, hk, hv, hdo = [t.cpu().pin_memory() for t in (q, k, v, do)]
    outs_host = [torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    rows = w["batch"]
    slots = [[torch.empty_like(t) for t in (q, k, v, do)] for _ in range(2)]
    slot_free = [[None] * rows for _ in range(2)]
    counter = [0]

    def e2e_step():
      main = torch.cuda.current_stream(dev)
      i = counter[0] & 1
      counter[0] += 1
      for b in range(rows):
        qb, kb, vb, dob = (t[b:b + 1] for t in slots[i])
        with torch.cuda.stream(s_in):
          if slot_free[i][b] is not None:
            s_in.wait_event(slot_free[i][b])  # the step that last used this buffer has finished with it
          qb.copy_(hq[b:b + 1], non_blocking=True)
          kb.copy_(hk[b:b + 1], non_blocking=True)
          vb.copy_(hv[b:b + 1], non_blocking=True)
          qkv_in = torch.cuda.Event()
          qkv_in.record(s_in)
          dob.copy_(hdo[b:b + 1], non_blocking=True)
          do_in = torch.cuda.Event()
          do_in.record(s_in)
        main.wait_event(qkv_in)
        qd, kd, vd = (t.detach().requires_grad_(True) for t in (qb, kb, vb))
        seg_b = None if seg is None else splash.SegmentIds(seg[0][b:b + 1], seg[1][b:b + 1])
        out = kernel(qd, kd, vd, seg_b, logits_scale=SCALE)
        fwd_done = torch.cuda.Event()
        fwd_done.record(main)
        with torch.cuda.stream(s_out):
          s_out.wait_event(fwd_done)
          outs_host[0][b:b + 1].copy_(out.detach(), non_blocking=True)
          out.record_stream(s_out)
        main.wait_event(do_in)
        out.backward(dob)
        bwd_done = torch.cuda.Event()
        bwd_done.record(main)
        slot_free[i][b] = bwd_done
        with torch.cuda.stream(s_out):
          s_out.wait_event(bwd_done)
          for dst, src in zip(outs_host[1:], (qd.grad, kd.grad, vd.grad)):
            dst[b:b + 1].copy_(src, non_blocking=True)
            src.record_stream(s_out)

    def e2e_run(n):
      for _ in range(n):
        e2e_step()
      torch.cuda.current_stream(dev).wait_stream(s_out)

    e2e_steps = max(10, min(args.steps, 20))
    ms_e2e = timed_steps(lambda: e2e_run(e2e_steps), 1, 1) / e2e_steps
    h2d = sum(t.numel() * 2 for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * 2 for t in outs_host)
    e2e = {"value": flops / ms_e2e / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "steps": e2e_steps,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "pinned_copy": pinned_copy_gbs(dev),
           "note": "pinned host buffers in and out; copies per batch row on side streams, double-buffered across steps"}
    del hq, hk, hv, hdo, outs_host, slots

  # ---- per-kernel times and the roofline of the dominant kernel
  peak, peak_sustained, peak_src = measured_peaks()
  kt = per_kernel_times(kernel, q, k, v, do, seg)
  # Split of the 14*D FLOPs per live pair: forward 4*D (QK^T, PV); backward 10*D — all of it in the
  # fused kernel, or, in the split form, dq kernel 4*D (dQ = dS K plus half of the shared S / dP
  # recomputation) and dkv kernel 6*D (dK, dV plus the other half).
  shares = {"fwd": 4, "dq": 4, "dkv": 6, "bwd_fused": 10}
  dominant = max((n for n in kt if n in shares), key=lambda n: kt[n])
  share = shares[dominant]
  k_flops = share * D * w["q_heads"] * n_live
  achieved = k_flops / kt[dominant] / 1e9
  roofline = {
      "kernel": {"fwd": "splash_fwd_kernel", "dq": "splash_dq_kernel", "dkv": "splash_dkv_kernel<.,false>",
                 "bwd_fused": "splash_dkv_kernel<.,true>"}[dominant],
      "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
      "peak_source": f"{peak_src} bf16 burst", "traffic": KERNEL_TRAFFIC_BYTES_C2.get(dominant) if wname == "c2" else None,
      "backward_form": args.bwd,
      "kernel_ms": kt,
      "whole_step_frac_of_peak": value / peak, "whole_step_frac_of_sustained": value / peak_sustained,
      "whole_step_frac_of_datasheet_2250": value / 2250.0,
  }

  line = {
      "metric": "splash fwd+bwd TFLOP/s (masked FLOPs)", "value": value, "unit": "TFLOP/s", "n_gpus": 1,
      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
      "scaling_note": "single GPU; the N > 1 runs of this script time another workload (c4, one long sequence split "
                      "over the GPUs, strong scaling) and carry their own one-GPU time in cp.single_gpu_ms_per_step",
      "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
      "config": {"workload": wname, **{k_: w[k_] for k_ in ("batch", "q_heads", "kv_heads", "seq", "mask")},
                 "head_dim": D, "n_live_pairs": n_live, "flops_per_step": flops,
                 "l2": l2_note(w)},
      "clocks": clocks, "e2e": e2e, "gpu_launches": 4 * args.steps, "roofline": roofline,
  }
  line["maskinfo_build_ms"] = maskinfo_build_times(w)
  if wname == "c2" and not args.no_other_workloads:
    # short runs of the other single-GPU workloads, so their numbers come from the same record
    del q, k, v, do
    torch.cuda.empty_cache()
    short = argparse.Namespace(**{**vars(args), "steps": 5, "warmup": 3, "no_e2e": True, "no_cpu_baseline": True,
                                  "no_other_workloads": True})
    other = {}
    for name, fn in (("c3", run_single_gpu), ("c5", run_fp8_prefill)):
      sub = fn(short, WORKLOADS[name], name, emit=False)
      other[name] = {"metric": sub["metric"], "value": sub["value"], "unit": sub["unit"], "ms_per_step": sub["ms_per_step"],
                     "steps": sub["steps"], "dtype": sub["dtype"], "clocks": sub["clocks"],
                     "frac_of_peak": sub["roofline"]["frac"], "peak": sub["roofline"]["peak"],
                     "peak_source": sub["roofline"]["peak_source"], "config": sub["config"],
                     "kernel_ms": sub["roofline"].get("kernel_ms")}
      torch.cuda.empty_cache()
    other["wide_head_dims"] = wide_head_dims(dev)
    line["other_workloads"] = other
  if not args.no_cpu_baseline:
    line["cpu_baseline"] = cpu_baseline(w)
  if emit:
    print(json.dumps(line), flush=True)
  return line


def wide_head_dims(dev, steps: int = 5) -> dict:
  """The head dims above 128 the reference's splash microbenchmarks quote — (q k, v) = (192, 128) and
  (256, 256); causal, batch 1, 32 q heads, 8 kv heads, S = 8192 — forward and backward in mask-counted
  TFLOP/s (forward 2 * d_qk + 2 * d_v FLOPs per live pair, backward 2 * (3 * d_qk + 2 * d_v))."""
  from tokamax_b200 import splash_attention_kernel as splash
  from tokamax_b200 import splash_attention_mask as mask_lib

  s, hq, hkv = 8192, 32, 8
  kernel = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  peak, _, _ = measured_peaks()
  live = hq * (s * (s + 1) // 2)
  out = {}
  for d_qk, d_v in ((192, 128), (256, 256)):
    g = torch.Generator(device=dev).manual_seed(7000 + d_qk)
    q, k, v, do = (torch.randn(1, h, s, d, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                   for h, d in ((hq, d_qk), (hkv, d_qk), (hkv, d_v), (hq, d_v)))
    scale = 1 / math.sqrt(d_qk)
    with torch.no_grad():
      ms_f = timed_steps(lambda: kernel(q, k, v, logits_scale=scale), steps, 3)

    def fwd_bwd():
      qd, kd, vd = (t.detach().requires_grad_(True) for t in (q, k, v))
      kernel(qd, kd, vd, logits_scale=scale).backward(do)

    ms_fb = timed_steps(fwd_bwd, steps, 3)
    f_fwd, f_bwd = live * (2 * d_qk + 2 * d_v), live * 2 * (3 * d_qk + 2 * d_v)
    out[f"{d_qk}_{d_v}"] = {
        "fwd_ms": ms_f, "fwd_tflops": f_fwd / ms_f / 1e9, "fwd_frac_of_peak": f_fwd / ms_f / 1e9 / peak,
        "bwd_ms": ms_fb - ms_f, "bwd_tflops": f_bwd / (ms_fb - ms_f) / 1e9,
        "bwd_frac_of_peak": f_bwd / (ms_fb - ms_f) / 1e9 / peak,
        "fwd_bwd_ms": ms_fb, "fwd_bwd_tflops": (f_fwd + f_bwd) / ms_fb / 1e9}
  kernel.check_errors()
  out["config"] = {"batch": 1, "q_heads": hq, "kv_heads": hkv, "seq": s, "mask": "causal"}
  return out


def run_fp8_prefill(args, w, wname, emit=True):
  """Forward only on block-scaled e4m3 Q/K/V (scales per 128-token tile), bf16 output."""
  from tokamax_b200 import fp8

  dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
  torch.cuda.set_device(dev)
  kernel = make_kernel(w)
  n_live = live_pairs(w, None)
  flops = 4 * D * w["q_heads"] * n_live
  q, k, v, _ = device_inputs(w, dev)
  qq, kq, vq = (fp8.quantize_e4m3(t) for t in (q, k, v))

  def step():
    return fp8.splash_fwd_fp8(kernel, qq, kq, vq, logits_scale=SCALE)

  def step_bf16():
    with torch.no_grad():
      return kernel(q, k, v, logits_scale=SCALE)

  sampler = ClockSampler(dev.index or 0)
  sampler.start()
  for _ in range(args.warmup):
    step()
  torch.cuda.synchronize()
  sampler.mark()
  ms = timed_steps(step, args.steps, 0)
  clocks = sampler.stop()
  kernel.check_errors()
  ms_bf16 = timed_steps(step_bf16, max(3, args.steps // 3), 2)
  # the variant that keeps the probabilities 16 bits wide (meets the bf16 forward's output bound)
  ms_p16 = timed_steps(lambda: fp8.splash_fwd_fp8(kernel, qq, kq, vq, logits_scale=SCALE, p_format="f16"),
                       max(3, args.steps // 3), 2)
  kernel.check_errors()
  value = flops / ms / 1e9

  e2e = None
  if not args.no_e2e:
    host = [t.cpu().pin_memory() for pair in (qq, kq, vq) for t in (pair.data.view(torch.uint8), pair.scale)]
    o_host = torch.empty((w["batch"], w["q_heads"], w["seq"], D), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
      d = [t.to(dev, non_blocking=True) for t in host]
      ts = [fp8.Fp8Tensor(d[2 * i].view(torch.float8_e4m3fn), d[2 * i + 1]) for i in range(3)]
      o_host.copy_(fp8.splash_fwd_fp8(kernel, *ts, logits_scale=SCALE), non_blocking=True)

    e2e_steps = max(10, min(args.steps, 20))
    ms_e2e = timed_steps(e2e_step, e2e_steps, 2)
    e2e = {"value": flops / ms_e2e / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "steps": e2e_steps,
           "pinned_copy": pinned_copy_gbs(dev),
           "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host),
           "d2h_bytes_per_step": o_host.numel() * 2}

  peak, _, peak_src = measured_peaks()
  fp8_peak = fp8_gemm_peak_tflops(dev)
  if fp8_peak is not None:
    peak8, peak8_src = fp8_peak, "e4m3 GEMM (torch._scaled_mm, 8192^3) measured in this run"
  else:
    peak8, peak8_src = 2 * peak, f"2 x {peak_src} bf16 burst (an e4m3 GEMM could not be timed here)"
  line = {
      "metric": "splash fp8 forward TFLOP/s (masked FLOPs)", "value": value, "unit": "TFLOP/s", "n_gpus": 1,
      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
      "vs_baseline": None, "dtype": "f8e4m3", "data": "synthetic",
      "config": {"workload": wname, **{k_: w[k_] for k_ in ("batch", "q_heads", "kv_heads", "seq", "mask")},
                 "head_dim": D, "n_live_pairs": n_live, "flops_per_step": flops,
                 "l2": "inputs (168 MB of e4m3 plus a 537 MB output) are larger than the 126 MB L2"},
      "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps,
      "roofline": {"kernel": "splash_fwd_kernel<true>", "bound": "tensor", "achieved": value, "peak": peak8,
                   "unit": "TFLOP/s", "frac": value / peak8, "peak_source": peak8_src,
                   "traffic": None, "bf16_forward_same_shape_tflops": flops / ms_bf16 / 1e9,
                   "p_f16_variant_tflops": flops / ms_p16 / 1e9},
  }
  if emit:
    print(json.dumps(line), flush=True)
  return line


def run_context_parallel(args, w, wname):
  import torch.distributed as dist
  from tokamax_b200 import ulysses

  rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
  local = int(os.environ.get("LOCAL_RANK", rank))
  dev = torch.device("cuda", local)
  torch.cuda.set_device(dev)
  # More NCCL channels for the point-to-point transfers an all-to-all is made of: on two B200s the
  # default moved 405 GB/s per direction, these settings 569 GB/s (a user's own settings win).
  for name, value in (("NCCL_MIN_NCHANNELS", "32"), ("NCCL_MIN_P2P_NCHANNELS", "64"), ("NCCL_MAX_P2P_NCHANNELS", "64")):
    os.environ.setdefault(name, value)
  dist.init_process_group("nccl", device_id=dev)
  kernel = make_kernel(w, args.bwd)
  s_loc = w["seq"] // world
  q, k, v, do = device_inputs(w, dev, seq_slice=s_loc)
  ring_mode = args.cp in ("ring", "ring_zigzag")
  if ring_mode:
    from tokamax_b200 import ring_attention
    from tokamax_b200 import splash_attention_mask as mask_lib
    if w["mask"] != "causal":
      raise SystemExit("--cp ring is wired for the causal workloads")
    cp = ring_attention.make_ring_attention(mask_lib.CausalMask((w["seq"], w["seq"])),
                                            layout="zigzag" if args.cp == "ring_zigzag" else "contiguous")
  else:
    exchange_used = args.exchange
    if args.exchange == "auto":
      # every rank must take the same branch: agree on whether the peer engine came up everywhere
      try:
        cp = ulysses.UlyssesSplashAttention(kernel, exchange="fused")
        cp.engine.exchange(torch.zeros(1, world, 128, D, dtype=torch.bfloat16, device=dev), True, "probe")
        ok_here = 1.0
      except Exception as e:  # pylint: disable=broad-except
        ok_here, why = 0.0, f"{type(e).__name__}: {e}"
      flag = torch.tensor([ok_here], device=dev)
      dist.all_reduce(flag, op=dist.ReduceOp.MIN)
      if flag.item() == 1.0:
        exchange_used = "fused"
      else:
        exchange_used = "nccl (peer exchange unavailable" + (f": {why})" if ok_here == 0.0 else " on another rank)")
        cp = ulysses.UlyssesSplashAttention(kernel, exchange="nccl")
    elif args.exchange == "fused-o":  # the output from the forward kernel, the gradients by the copy kernel
      cp = ulysses.UlyssesSplashAttention(kernel, exchange="fused", fuse_gradients=False)
    else:
      cp = ulysses.UlyssesSplashAttention(kernel, exchange=args.exchange)
  n_live = live_pairs(w, None)
  flops = 14 * D * w["q_heads"] * n_live

  def step():
    qd, kd, vd = q.detach().requires_grad_(True), k.detach().requires_grad_(True), v.detach().requires_grad_(True)
    out = cp(qd, kd, vd, logits_scale=SCALE)
    out.backward(do)

  def max_over_ranks(ms):
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()

  sampler = ClockSampler(local)
  sampler.start()
  for _ in range(args.warmup):
    step()
  dist.barrier()
  torch.cuda.synchronize()
  sampler.mark()
  ms = max_over_ranks(timed_steps(step, args.steps, 0, barrier=dist.barrier))
  clocks = sampler.stop()
  kernel.check_errors()
  if ring_mode:
    cp.check_errors()  # the ring runs its own per-pair kernels

  # exchange alone: the 4 + 4 all-to-alls of one step (q, k, v, o forward; do, dq, dk, dv backward)
  def exchanges(skip=()):
    engine = getattr(cp, "engine", None)
    run = (lambda t, s2h, tag: ulysses._run_exchange(t, None, s2h, engine, tag))  # pylint: disable=protected-access
    for name, t in (("q", q), ("k", k), ("v", v), ("do", do)):
      run(t, True, "bench." + name)
    qh = torch.empty((w["batch"], w["q_heads"] // world, w["seq"], D), dtype=q.dtype, device=dev)
    kh = torch.empty((w["batch"], w["kv_heads"] // world, w["seq"], D), dtype=q.dtype, device=dev)
    for name, t in (("o", qh), ("dq", qh), ("dk", kh), ("dv", kh)):
      if name not in skip:
        run(t, False, "bench." + name)
  a2a_ms = None if ring_mode else max_over_ranks(timed_steps(exchanges, 3, 1, barrier=dist.barrier))
  # "fused": the kernels store the output (and, with the fused backward, the gradients) straight into
  # the ranks that own the rows — o, dk, dv from the epilogues of long kernels, dq from the cast pass —
  # so only the input exchanges (q, k, v, do) stay in line with the kernels
  exposed_ms = a2a_ms
  if not ring_mode and getattr(cp, "fused", False):
    inside = ("o", "dq", "dk", "dv") if cp.fuse_gradients and not kernel.repeatable_dq else ("o",)
    exposed_ms = max_over_ranks(timed_steps(lambda: exchanges(skip=inside), 3, 1, barrier=dist.barrier))
  sent = 2 * (2 * ulysses.exchange_bytes_sent(q.shape, 2, world) + 2 * ulysses.exchange_bytes_sent(k.shape, 2, world))

  # end to end: each rank's sequence shard starts and ends in pinned host memory.  Copies run on two
  # side streams and are double-buffered across steps: while step n computes, step n+1's inputs come
  # in and step n-1's gradients go out; within a step dO follows q/k/v (the forward does not need
  # it) and the output leaves while the backward runs.
  e2e = None
  if not args.no_e2e:
    hq, hk, hv, hdo = [t.cpu().pin_memory() for t in (q, k, v, do)]
    outs_host = [torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    slots = [[torch.empty_like(t) for t in (q, k, v, do)] for _ in range(2)]
    slot_free = [None, None]
    counter = [0]

    def e2e_step():
      main = torch.cuda.current_stream(dev)
      i = counter[0] & 1
      counter[0] += 1
      a, b_, c, d_ = slots[i]
      with torch.cuda.stream(s_in):
        if slot_free[i] is not None:
          s_in.wait_event(slot_free[i])  # the step that last used this slot has finished with it
        a.copy_(hq, non_blocking=True)
        b_.copy_(hk, non_blocking=True)
        c.copy_(hv, non_blocking=True)
        qkv_in = torch.cuda.Event()
        qkv_in.record(s_in)
        d_.copy_(hdo, non_blocking=True)
        do_in = torch.cuda.Event()
        do_in.record(s_in)
      main.wait_event(qkv_in)
      qd, kd, vd = a.detach().requires_grad_(True), b_.detach().requires_grad_(True), c.detach().requires_grad_(True)
      out = cp(qd, kd, vd, logits_scale=SCALE)
      fwd_done = torch.cuda.Event()
      fwd_done.record(main)
      with torch.cuda.stream(s_out):
        s_out.wait_event(fwd_done)
        outs_host[0].copy_(out.detach(), non_blocking=True)
        out.record_stream(s_out)
      main.wait_event(do_in)
      out.backward(d_)
      bwd_done = torch.cuda.Event()
      bwd_done.record(main)
      slot_free[i] = bwd_done
      with torch.cuda.stream(s_out):
        s_out.wait_event(bwd_done)
        for dst, src in zip(outs_host[1:], (qd.grad, kd.grad, vd.grad)):
          dst.copy_(src, non_blocking=True)
          src.record_stream(s_out)

    def e2e_run(n):
      for _ in range(n):
        e2e_step()
      torch.cuda.current_stream(dev).wait_stream(s_out)

    e2e_steps = max(10, min(args.steps, 20))
    ms_e2e = max_over_ranks(timed_steps(lambda: e2e_run(e2e_steps), 1, 1, barrier=dist.barrier)) / e2e_steps
    e2e = {"value": flops / ms_e2e / 1e9, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "steps": e2e_steps,
           "h2d_bytes_per_step": world * sum(t.numel() * 2 for t in (hq, hk, hv, hdo)),
           "d2h_bytes_per_step": world * sum(t.numel() * 2 for t in outs_host),
           "pinned_copy_rank0_alone": pinned_copy_gbs(dev) if rank == 0 else None,
           "note": "per-rank pinned host buffers in and out; copies on side streams, double-buffered across steps"}
    del hq, hk, hv, hdo, outs_host, slots

  # the same workload on one GPU alone (all heads, no exchange), timed on rank 0 while the others
  # wait: the denominator-free way to read the scaling of THIS workload
  single_ms = None
  if not args.no_single_gpu_ref and not ring_mode:
    del q, k, v, do
    torch.cuda.empty_cache()
    if rank == 0:
      q1, k1, v1, do1 = device_inputs(w, dev)

      def step1():
        qd, kd, vd = q1.detach().requires_grad_(True), k1.detach().requires_grad_(True), v1.detach().requires_grad_(True)
        kernel(qd, kd, vd, logits_scale=SCALE).backward(do1)

      single_ms = timed_steps(step1, 3, 2)
      kernel.check_errors()
      del q1, k1, v1, do1
    dist.barrier()

  if rank == 0:
    peak, peak_sustained, peak_src = measured_peaks()
    value = flops / ms / 1e9
    line = {
        "metric": "splash fwd+bwd TFLOP/s (masked FLOPs)", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "scaling_note": "total work is fixed (one 131072-token sequence) and split over the GPUs; the N = 1 default "
                        "line of this script is a different workload (c2), so use cp.scaling_efficiency",
        "config": {"workload": wname, **{k_: w[k_] for k_ in ("batch", "q_heads", "kv_heads", "seq", "mask")},
                   "head_dim": D, "parallelism": f"{args.cp if ring_mode else 'ulysses'} cp{world}",
                   "exchange": None if ring_mode else exchange_used,
                   "n_live_pairs": n_live,
                   "flops_per_step": flops, "l2": "inputs are larger than the 126 MB L2"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": 4 * args.steps,
        "cp": {"tokens_per_s": w["batch"] * w["seq"] / (ms / 1e3), "a2a_ms_per_step": a2a_ms,
               "a2a_bytes_sent_per_gpu": None if ring_mode else sent,
               "a2a_gbs_per_direction": None if ring_mode else sent / a2a_ms / 1e6,
               "nvlink_nominal_gbs_per_direction": 900.0,
               "single_gpu_ms_per_step": single_ms,
               "scaling_efficiency": None if single_ms is None else single_ms / (world * ms),
               # the exchanges run in line with the kernels, so all of their time is exposed; with
               # --exchange fused the outputs' exchanges are part of the kernels and are left out
               "exposed_a2a_ms_per_step": exposed_ms,
               },
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peak_sustained, "unit": "TFLOP/s",
                     "frac": value / world / peak_sustained, "peak_source": f"{peak_src} bf16 sustained, per GPU",
                     "traffic": None},
    }
    print(json.dumps(line), flush=True)
  dist.barrier()
  dist.destroy_process_group()


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=30)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
  ap.add_argument("--workload", default="auto", choices=["auto", "c1", "c2", "c3", "c4", "c5", "wide"])
  ap.add_argument("--exchange", default="auto", choices=["auto", "nccl", "peer", "fused", "fused-o"],
                  help="Ulysses exchange: the library's own peer-store kernel over symmetric memory (peer), NCCL "
                       "all_to_all_single (nccl), or peer with nccl as the fallback if symmetric memory cannot be set up (auto)")
  ap.add_argument("--cp", default="ulysses", choices=["ulysses", "ring", "ring_zigzag"],
                  help="context-parallel scheme for N > 1 (ring: K/V rotate, causal load is unbalanced)")
  ap.add_argument("--bwd", default="fused", choices=["fused", "split"],
                  help="backward form: one fused kernel (dQ partials reduced in fp32) or separate dq / dkv kernels")
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--no-cpu-baseline", action="store_true")
  ap.add_argument("--no-single-gpu-ref", action="store_true",
                  help="N > 1: skip timing the same workload on rank 0 alone (cp.single_gpu_ms_per_step)")
  ap.add_argument("--no-other-workloads", action="store_true",
                  help="N = 1, c2: skip the short c3 / c5 runs reported under other_workloads")
  args = ap.parse_args()
  args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
  world = int(os.environ.get("WORLD_SIZE", "1"))
  wname = args.workload
  if wname == "auto":
    wname = "c2" if world == 1 else "c4"
  if wname == "wide":  # head dims (192, 128) and (256, 256): a side line, not a headline workload
    if args.impl != "ours" or world != 1 or not torch.cuda.is_available():
      raise SystemExit("--workload wide is a single-GPU run of this build's forward")
    print(json.dumps({"metric": "splash TFLOP/s (masked FLOPs), head dims above 128", "unit": "TFLOP/s",
                      "n_gpus": 1, "steps": args.steps, "dtype": "bf16", "data": "synthetic",
                      **wide_head_dims(torch.device("cuda", 0), max(args.steps, 1))}), flush=True)
    return
  w = WORKLOADS[wname]
  if args.impl == "reference":
    run_reference(args, w, wname)
    return
  if not torch.cuda.is_available():
    raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path for the kernels")
  if wname == "c5":
    if world != 1:
      raise SystemExit("c5 (fp8 prefill) is a single-GPU workload")
    run_fp8_prefill(args, w, wname)
  elif world == 1:
    run_single_gpu(args, w, wname)
  else:
    run_context_parallel(args, w, wname)


if __name__ == "__main__":
  main()
