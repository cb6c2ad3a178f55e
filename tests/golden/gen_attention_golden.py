"""Generates tests/golden/attention_golden.npz by running the REFERENCE's own dense attention oracle.

    SPLASH_REFERENCE_ROOT=<path to primatrix/tokamax> python tests/golden/gen_attention_golden.py

The reference's ``base.py`` (``attention_reference`` with residuals, ``attention_reference_vjp`` with
both ``backward_impl`` values) is loaded unmodified through oracle/ref_loader.py, where numpy stands
in for ``jax.numpy`` (JAX is not installed where this was generated; see
``ref_loader._install_numpy_jnp`` for what that changes: the order of fp32 summation, nothing
else).  Its outputs for every case of attention_cases.CASES are stored as float32; the CPU tests
compare the torch restatement ``oracle/attention_ref.py`` against them without a reference tree.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from oracle import ref_loader  # noqa: E402
import attention_cases as cases  # noqa: E402


def main():
  base = ref_loader.load_reference_base()
  store = {}
  for case in cases.CASES:
    q, k, v, do, mask, seg, sinks = cases.build(case)
    seg_ids = None if seg is None else base.SegmentIds(q=seg[0], kv=seg[1])
    kw = dict(is_mqa=case["mqa"], attn_logits_soft_cap=case["soft_cap"])
    o, res = base.attention_reference(q, k, v, mask, seg_ids, sinks, save_residuals=True, **kw)
    store[f"{case['name']}/o"] = o
    store[f"{case['name']}/logsumexp"] = res["logsumexp"]
    store[f"{case['name']}/max_logits"] = res["max_logits"]
    o_stored = cases.to_bf16(o)  # the kernels (and the reference's) take di from the stored output
    for impl in ("flash", "vanilla") if case["name"] in cases.VANILLA_TOO else ("flash",):
      dq, dk, dv, dsinks = base.attention_reference_vjp(do, q, k, v, mask, seg_ids, sinks, o_stored, res["logsumexp"],
                                                        backward_impl=impl, **kw)
      for name, value in (("dq", dq), ("dk", dk), ("dv", dv), ("dsinks", dsinks)):
        if value is not None:
          store[f"{case['name']}/{impl}/{name}"] = np.asarray(value, dtype=np.float32)
    print(case["name"], "ok", flush=True)
  out = os.path.join(HERE, "attention_golden.npz")
  np.savez_compressed(out, **store)
  print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
  main()
