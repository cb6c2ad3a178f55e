"""The kernel module's public surface, name by name, against the reference's
(tokamax/_src/ops/experimental/tpu/splash_attention/splash_attention_kernel.py: SplashConfig :114-196,
QKVLayout :103-105, get_kernel_name :86-96, from_head_minor :108-111, the make_* factories
:2070-2237, SplashAttentionKernel :2002-2067).  The lists below were read off the reference's
source; a reference call site must find every name, field, default and parameter it uses.
"""
import dataclasses
import inspect

import pytest

from tokamax_b200 import splash_attention_kernel as splash

# (field, default as written in the reference; None = required)
CONFIG_FIELDS = [
    ("block_q", None), ("block_kv", None), ("block_kv_compute", "None"), ("block_q_dkv", "None"),
    ("block_kv_dkv", "None"), ("block_kv_dkv_compute", "None"), ("block_q_dq", "None"), ("block_kv_dq", "None"),
    ("use_fused_bwd_kernel", "True"), ("num_stacked_q_heads", "1"), ("q_layout", "QKVLayout.HEAD_DIM_MINOR"),
    ("k_layout", "QKVLayout.HEAD_DIM_MINOR"), ("v_layout", "QKVLayout.HEAD_DIM_MINOR"), ("fwd_cost_estimate", "None"),
    ("bwd_cost_estimate", "None"), ("residual_checkpoint_name", "None"), ("attn_logits_soft_cap", "None"),
    ("fuse_reciprocal", "True"), ("use_base2_exp", "True"), ("max_logit_const", "None"), ("interpret", "False"),
    ("dq_reduction_steps", "None"), ("use_experimental_scheduler", "False"),
]
FACTORIES = ["make_splash_mha", "make_splash_mqa", "make_splash_mha_single_device", "make_splash_mqa_single_device",
             "make_dynamic_splash_mha", "make_dynamic_splash_mqa"]
FACTORY_KEYWORDS = ["config", "save_residuals", "mask_value", "downcast_smem_data", "partial_mask_blocks_dtype"]
KERNEL_METHODS = ["__call__", "manual_sharding_spec", "tree_flatten", "tree_unflatten"]


def test_config_fields_and_defaults():
  fields = dataclasses.fields(splash.SplashConfig)
  assert [f.name for f in fields] == [name for name, _ in CONFIG_FIELDS]
  namespace = {"QKVLayout": splash.QKVLayout, "None": None, "True": True, "False": False}
  for f, (name, default) in zip(fields, CONFIG_FIELDS):
    if default is None:
      assert f.default is dataclasses.MISSING, name
    else:
      assert f.default == eval(default, namespace), name  # pylint: disable=eval-used
  assert [m.name for m in splash.QKVLayout] == ["HEAD_DIM_MINOR", "SEQ_MINOR"]
  assert isinstance(splash.SplashConfig.get_default(), splash.SplashConfig)


def test_helpers():
  assert splash.get_kernel_name(True, False, True, "dkv") == "splash_mqa_dkv_segmented_no_residuals"
  assert splash.get_kernel_name(False, True, False, "fwd") == "splash_mha_fwd_residuals"
  with pytest.raises(AssertionError):
    splash.get_kernel_name(False, True, False, "dq")  # residuals exist in the forward only
  assert list(inspect.signature(splash.get_kernel_name).parameters) == ["is_mqa", "save_residuals", "is_segmented", "phase"]
  assert splash.from_head_minor((2, 8, 128), splash.QKVLayout.SEQ_MINOR) == (2, 128, 8)
  assert splash.from_head_minor((2, 8, 128), splash.QKVLayout.HEAD_DIM_MINOR) == (2, 8, 128)
  assert list(inspect.signature(splash.from_head_minor).parameters) == ["vals", "layout"]
  for name in ("MaskInfo", "SegmentIds", "DEFAULT_MASK_VALUE"):
    assert hasattr(splash, name), name


@pytest.mark.parametrize("name", FACTORIES)
def test_factories_take_the_reference_keywords(name):
  params = inspect.signature(getattr(splash, name)).parameters
  assert list(params)[0] == "mask"
  for kw in FACTORY_KEYWORDS:
    assert kw in params or any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()), (name, kw)
  if "dynamic" not in name and "single_device" not in name:
    assert "q_seq_shards" in params, name


def test_kernel_object_methods():
  for name in KERNEL_METHODS:
    assert callable(getattr(splash.SplashAttentionKernel, name)), name
  init = list(inspect.signature(splash.SplashAttentionKernel.__init__).parameters)
  assert init[:3] == ["self", "fwd_mask_info", "dkv_mask_info"]
