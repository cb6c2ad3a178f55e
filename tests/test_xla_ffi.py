"""The XLA custom-call adapter without XLA: what can be checked on a CPU.

* the normal build (no xla/ffi/api/ffi.h on the include path) carries no handler and is otherwise
  unchanged;
* every operand / result / attribute the handlers declare maps onto a field of SplashFwdArgs /
  SplashBwdArgs, and every field of those structs is filled by some handler argument (or derived
  from one);
* the adapter compiles against a stand-in of the FFI header and, called with fake buffers, hands
  the right pointers, strides and attributes to the C ABI (tests/xla_ffi_stub/driver.cc);
* the host-side call plan built from a kernel object lines up with the handler signature.
The handlers themselves have not run under XLA: JAX is not installed where these tests run.
"""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

from tokamax_b200 import _native
from tokamax_b200 import splash_attention_kernel as splash
from tokamax_b200 import splash_attention_mask as mask_lib
from tokamax_b200 import xla_ffi

HERE = os.path.dirname(os.path.abspath(__file__))


def _leaf_fields(struct, prefix=""):
  out = []
  for name, ctype in struct._fields_:  # pylint: disable=protected-access
    if isinstance(ctype, type) and issubclass(ctype, C.Structure) and ctype is not _native.SplashTensor:
      out += _leaf_fields(ctype, prefix + name + ".")
    else:
      out.append(prefix + name)
  return out


def test_normal_build_has_no_handlers_and_reports_so():
  lib = _native.lib()
  assert lib.splash_xla_ffi_compiled() == 0
  for sym in xla_ffi.HANDLER_SYMBOLS.values():
    assert not hasattr(lib, sym)
  assert lib.splash_xla_ffi_signature(7) == b""


@pytest.mark.parametrize("which,struct", [(xla_ffi.FWD, _native.SplashFwdArgs), (xla_ffi.BWD, _native.SplashBwdArgs)])
def test_handler_arguments_cover_the_args_struct_field_for_field(which, struct):
  sig = xla_ffi.signature(which)
  fields = set(_leaf_fields(struct))
  filled = set()
  for group in ("operands", "results", "attrs"):
    for name, _ in sig[group]:
      path = xla_ffi.field_path(name, which)
      if path is None:
        continue
      for p in path.split("+"):
        assert p in fields, (name, p)
        filled.add(p)
  # derived inside the handler from the sizes of the arrays it is given, or fixed
  derived = {f"{s}.{leaf}" for s in ("sched", "sched_dq", "sched_dkv") for leaf in ("n_rows", "n_entries")}
  derived |= {"workspace_bytes", "launch_mask"}
  # second destinations of outputs in other ranks' memory: not reachable from a single-device custom call, left zero
  derived |= {f"{out}_peer.{leaf}" for out in ("o", "dq", "dk", "dv")
              for leaf in ("ptrs", "base_bytes", "rows_per_peer", "stride_b", "stride_h", "stride_s", "head0")}
  assert fields - filled <= derived, sorted(fields - filled - derived)
  names = [n for g in ("operands", "results", "attrs") for n, _ in sig[g]]
  assert len(names) == len(set(names))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")
def test_adapter_compiles_against_a_stub_of_the_ffi_header_and_fills_the_structs(tmp_path):
  stub = os.path.join(HERE, "xla_ffi_stub")
  exe = str(tmp_path / "ffi_driver")
  build = subprocess.run(["g++", "-std=c++17", "-I", stub, "-o", exe, os.path.join(stub, "driver.cc")],
                         capture_output=True, text=True)
  assert build.returncode == 0, build.stderr
  run = subprocess.run([exe], capture_output=True, text=True)
  assert run.returncode == 0 and run.stdout.strip() == "OK", run.stdout + run.stderr


def test_call_plan_follows_the_signature():
  s = 512
  kernel = splash.make_splash_mha(mask_lib.LocalMask((s, s), (100, 0), 0) & mask_lib.CausalMask((s, s)), q_seq_shards=1)
  for which in (xla_ffi.FWD, xla_ffi.BWD):
    sig = xla_ffi.signature(which)
    plan = xla_ffi.call_plan(kernel, which, scale=0.125, layout=xla_ffi.LAYOUT_BSHD)
    assert [n for n, _ in plan["operands"]] == [n for n, _ in sig["operands"]]
    assert list(plan["attrs"]) == [n for n, _ in sig["attrs"]]
    assert plan["results"] == [n for n, _ in sig["results"]]
    ops = dict(plan["operands"])
    for name in ("q", "k", "v"):
      assert ops[name] is None  # supplied at run time
    prefix = "sched" if which == xla_ffi.FWD else "dkv"
    row_ptr, entries = ops[f"{prefix}_row_ptr"], ops[f"{prefix}_entries"]
    assert row_ptr.dtype == np.int32 and row_ptr[0] == 0 and len(entries) == 4 * row_ptr[-1]
    assert ops[f"{prefix}_partial_mask_blocks"].dtype == np.int8 and ops[f"{prefix}_partial_mask_blocks"].size > 0
    assert ops[f"{prefix}_row_end"].size == 0 and ops["q_sequence"].size == 0
    assert plan["attrs"]["layout"] == 1 and plan["attrs"]["scale"].dtype == np.float32
    assert plan["attrs"]["mask_kind"] == 0  # a composed mask has no in-kernel mask function
  causal = splash.make_splash_mha(mask_lib.CausalMask((s, s)), q_seq_shards=1)
  plan = xla_ffi.call_plan(causal, xla_ffi.BWD, scale=1.0, fused_backward=False)
  assert plan["attrs"]["mask_kind"] == 1 and plan["attrs"]["flags"] == 0


def test_jax_backend_needs_jax_and_says_so():
  try:
    import jax  # noqa: F401  pylint: disable=unused-import,g-import-not-at-top
    pytest.skip("jax is installed here")
  except ImportError:
    pass
  with pytest.raises(ImportError, match="jax"):
    import tokamax_b200.jax_backend  # noqa: F401  pylint: disable=unused-import,g-import-not-at-top


def test_autotuning_cache_entries_are_in_the_reference_format():
  """<device kind>/<snake-cased op class>.json: bound arguments (JSON) -> config (JSON) -> timings
  (reference tokamax/_src/autotuning/cache.py:72-112 and its shipped data files)."""
  import json
  import re

  op_name = re.sub(r"(?!^)([A-Z])", r"_\1", "CudaSm100SplashAttention").lower()
  root = os.path.join(os.path.dirname(HERE), "tokamax_b200", "data", "autotuning", "nvidia_b200")
  path = os.path.join(root, f"{op_name}.json")
  assert os.path.isfile(path), path
  data = json.load(open(path))
  assert data
  for key, configs in data.items():
    bound = json.loads(key)
    assert {"q", "k", "v", "mask", "logits_scale", "return_residuals"} <= set(bound)
    assert re.fullmatch(r"bf16\[\d+,\d+,\d+,(128|192|256)\]", bound["q"])
    for cfg, timing in configs.items():
      assert set(json.loads(cfg)) == {"block_q", "block_kv"}
      assert {"compile_time_ms", "lower_time_ms", "evaluation_times_ms", "metadata"} <= set(timing)
      assert all(t > 0 for t in timing["evaluation_times_ms"])


def test_jax_backend_overrides_have_the_reference_signatures():
  """`_fwd` of the backend and of its vjp, parameter by parameter, against the methods they
  override (tokamax/_src/ops/attention/base.py:564-584 and :813-843; the lists were read off the
  reference's source).  The module is parsed, not imported: it needs JAX."""
  import ast

  fwd = ["self", "q", "k", "v", "precision", "logits_dtype", "logits_scale", "bias", "logits_soft_cap", "mask",
         "dropout_mask", "dropout_rate", "paging_info", "q_indices", "k_indices", "normalize_output",
         "return_residuals", "config"]
  vjp = ["self", "residuals", "out", "dout"] + fwd[1:]
  path = os.path.join(os.path.dirname(HERE), "tokamax_b200", "jax_backend.py")
  tree = ast.parse(open(path).read())
  found = {}
  for node in tree.body:
    if isinstance(node, ast.ClassDef):
      for item in node.body:
        if isinstance(item, ast.FunctionDef) and item.name == "_fwd":
          a = item.args
          found[node.name] = [x.arg for x in a.posonlyargs + a.args] + [x.arg for x in a.kwonlyargs]
  assert found == {"CudaSm100SplashAttention": fwd, "CudaSm100SplashAttentionVjp": vjp}
  names = {n.name for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef))}
  assert {"Config", "register"} <= names
