"""Loads the reference's own numpy MaskInfo code without JAX.  TEST INFRASTRUCTURE ONLY.

The reference's ``splash_attention_mask.py`` is pure numpy and ``splash_attention_mask_info.py``
only touches JAX in ``find_bounds`` and ``_process_dynamic_mask``; with a stub ``jax`` package
pre-seeded in ``sys.modules`` both load and ``process_mask`` / ``process_mask_dkv`` run
unmodified.  This works only where a checkout of the reference is present and the environment
variable SPLASH_REFERENCE_ROOT points at it; it is used to generate ``tests/golden/maskinfo_*.npz`` and to run the reference's MaskInfo test-suite
against the oracle restatement and against the product's builder.

Nothing here copies reference sources: modules are loaded from where they lie.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import types

REFERENCE_ROOT = os.environ.get("SPLASH_REFERENCE_ROOT", "")  # unset: available() is False
_SA = "tokamax/_src/ops/experimental/tpu/splash_attention"
_PKG = "tokamax._src.ops.experimental.tpu.splash_attention"


def available() -> bool:
  return bool(REFERENCE_ROOT) and os.path.isfile(os.path.join(REFERENCE_ROOT, _SA, "splash_attention_mask_info.py"))


def _install_jax_stub() -> None:
  if "jax" in sys.modules and not getattr(sys.modules["jax"], "_splash_stub", False):
    return  # a real jax is importable; use it
  import numpy as np

  jax = types.ModuleType("jax")
  jax._splash_stub = True
  jax.Array = np.ndarray
  jax.jit = lambda f=None, **kw: f if f is not None else (lambda g: g)
  jax.default_backend = lambda: "cpu"
  jnp = types.ModuleType("jax.numpy")
  for name in ("isfinite", "roll", "arange", "any", "all", "where", "argwhere", "array", "int32"):
    setattr(jnp, name, getattr(np, name))
  try:
    import ml_dtypes

    jnp.bfloat16 = ml_dtypes.bfloat16
  except ImportError:
    pass
  lax = types.ModuleType("jax.lax")
  typing_mod = types.ModuleType("jax.typing")
  typing_mod.DTypeLike = object
  sharding = types.ModuleType("jax.sharding")
  sharding.PartitionSpec = tuple
  config = types.SimpleNamespace(parse_flags_with_absl=lambda *a, **k: None, update=lambda *a, **k: None)
  jax.numpy, jax.lax, jax.typing, jax.sharding, jax.config = jnp, lax, typing_mod, sharding, config
  sys.modules.update({"jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.typing": typing_mod,
                      "jax.sharding": sharding})


def _load(name: str):
  full = f"{_PKG}.{name}"
  if full in sys.modules:
    return sys.modules[full]
  parts = _PKG.split(".")
  for i in range(1, len(parts) + 1):
    pkg = ".".join(parts[:i])
    if pkg not in sys.modules:
      mod = types.ModuleType(pkg)
      mod.__path__ = []
      sys.modules[pkg] = mod
  spec = importlib.util.spec_from_file_location(full, os.path.join(REFERENCE_ROOT, _SA, name + ".py"))
  mod = importlib.util.module_from_spec(spec)
  sys.modules[full] = mod
  spec.loader.exec_module(mod)
  return mod


def load_reference():
  """Returns ``(mask_lib, mask_info_lib)`` — the reference's own modules."""
  if not available():
    raise FileNotFoundError(f"reference tree not found under {REFERENCE_ROOT}")
  _install_jax_stub()
  return _load("splash_attention_mask"), _load("splash_attention_mask_info")


def _install_numpy_jnp() -> None:
  """Gives the stub ``jax`` what the reference's dense attention oracle (base.py:74-285) calls, with
  numpy doing the arithmetic: the ``jnp`` functions it uses (same names and semantics in numpy;
  ``einsum`` drops ``preferred_element_type``, whose fp32 the fp32 operands already give), ``jax.jit``
  as the identity and ``jax.vmap`` as a Python loop over axis 0 that stacks the results leaf by leaf.
  The reference's code then runs unmodified; what differs from a run under XLA is the order of fp32
  summation inside einsum / sum, nothing else."""
  import numpy as np

  jax = sys.modules["jax"]
  if not getattr(jax, "_splash_stub", False) or getattr(jax, "_splash_numpy_jnp", False):
    return
  jnp = sys.modules["jax.numpy"]
  for name in ("logical_and", "tanh", "maximum", "exp", "log", "sum", "repeat", "float32", "where"):
    setattr(jnp, name, getattr(np, name))
  jnp.einsum = lambda spec, *ops, preferred_element_type=None, **kw: np.einsum(spec, *ops, **kw)

  def stack(items):
    first = items[0]
    if first is None:
      return None
    if isinstance(first, dict):
      return {k: stack([it[k] for it in items]) for k in first}
    if isinstance(first, tuple):
      return tuple(stack([it[i] for it in items]) for i in range(len(first)))
    return np.stack([np.asarray(it) for it in items])

  def vmap(fn, in_axes=0):
    def mapped(*args):
      axes = in_axes if isinstance(in_axes, (tuple, list)) else (in_axes,) * len(args)
      n = next(np.shape(a)[0] for a, ax in zip(args, axes) if ax == 0 and a is not None)
      return stack([fn(*[(a[i] if ax == 0 and a is not None else a) for a, ax in zip(args, axes)]) for i in range(n)])
    return mapped

  jax.vmap = vmap
  jax._splash_numpy_jnp = True


def load_reference_base():
  """The reference's ``base.py`` (its dense attention oracle ``attention_reference`` /
  ``attention_reference_vjp``), loaded unmodified and runnable on numpy arrays; see
  :func:`_install_numpy_jnp` for what stands in for JAX."""
  if not available():
    raise FileNotFoundError(f"reference tree not found under {REFERENCE_ROOT}")
  load_reference()       # (installs the stub jax)
  _install_numpy_jnp()   # before base.py binds `jnp`
  return _load("base")


def run_reference_mask_tests(mask_module=None, mask_info_module=None, verbosity: int = 0):
  """Runs the reference's ``splash_attention_mask_test.py`` and returns the unittest result.

  With ``mask_module`` / ``mask_info_module`` given, the test module's ``mask_lib`` /
  ``mask_info_lib`` aliases are pointed at them, turning the reference's golden-vector suite
  into an acceptance test of another implementation.  The TPU-only ``skipTest`` in ``setUp`` is
  neutralised (the tests themselves are pure numpy).
  """
  import unittest

  load_reference()
  _load("base")
  _load("splash_attention_test_utils")
  test_mod = _load("splash_attention_mask_test")
  if mask_module is not None:
    test_mod.mask_lib = mask_module
  if mask_info_module is not None:
    test_mod.mask_info_lib = mask_info_module
  for cls_name in ("SplashAttentionMaskTest", "SplashAttentionMaskInfoTest"):
    cls = getattr(test_mod, cls_name, None)
    if cls is not None:
      cls.setUp = lambda self: None
  suite = unittest.defaultTestLoader.loadTestsFromModule(test_mod)
  return unittest.TextTestRunner(verbosity=verbosity, stream=open(os.devnull, "w")).run(suite)
