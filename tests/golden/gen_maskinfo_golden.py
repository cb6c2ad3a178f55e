"""Generates tests/golden/maskinfo_golden.npz by running the REFERENCE's own MaskInfo builder.

Run where a checkout of the reference is present, pointing SPLASH_REFERENCE_ROOT at it:

    SPLASH_REFERENCE_ROOT=<path to primatrix/tokamax> python tests/golden/gen_maskinfo_golden.py

For every case of maskinfo_cases.CASES the reference's ``process_mask`` and ``process_mask_dkv``
(loaded unmodified through oracle/ref_loader.py) are called; each MaskInfo field is stored either
in full or, for the large cases, as ``sha256(dtype, shape, bytes)``.  ``None`` fields are recorded
in the ``__none__`` list.  The committed .npz is what the CPU tests compare the oracle restatement
and the native builder against, so those tests need no reference tree.
"""
import hashlib
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from oracle import ref_loader  # noqa: E402
import maskinfo_cases as cases  # noqa: E402


def digest(a: np.ndarray) -> np.ndarray:
  h = hashlib.sha256()
  h.update(str(a.dtype).encode())
  h.update(str(a.shape).encode())
  h.update(np.ascontiguousarray(a).tobytes())
  return np.frombuffer(h.digest(), dtype=np.uint8).copy()


def main():
  ref_mask, ref_mi = ref_loader.load_reference()
  store, none_fields, meta = {}, [], {}
  for case in cases.CASES:
    t0 = time.time()
    mask = cases.build_mask(case["mask"], ref_mask)
    kw = dict(downcast_smem_data=case["downcast"], q_seq_shards=case["q_shards"],
              kv_seq_shards=case["kv_shards"])
    fwd, fn = ref_mi.process_mask(mask, tuple(case["block"]), **kw)
    dkv, _ = ref_mi.process_mask_dkv(mask, tuple(case["block"]), return_dynamic_grid=case["dkv_dynamic"], **kw)
    for tag, info in (("fwd", fwd), ("dkv", dkv)):
      for field in cases.FIELDS:
        key = f"{case['name']}/{tag}/{field}"
        value = getattr(info, field)
        if value is None:
          none_fields.append(key)
        elif case["digest"]:
          store[key] = digest(np.asarray(value))
        else:
          store[key] = np.asarray(value)
    meta[case["name"]] = dict(has_mask_function=fn is not None, seconds=round(time.time() - t0, 3))
    print(case["name"], meta[case["name"]], flush=True)
  store["__none__"] = np.array(json.dumps(none_fields))
  store["__meta__"] = np.array(json.dumps(meta))
  out = os.path.join(HERE, "maskinfo_golden.npz")
  np.savez_compressed(out, **store)
  print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
  main()
