"""ctypes binding of ``libsplash_b200.so`` (declared in ``include/splash_b200.h``).

The library is built in-tree by :func:`build` (``nvcc`` for sm_100a) and loaded from
``tokamax_b200/lib``.  There is no fallback: if the library is missing or a call returns a
non-zero status the caller gets an exception.
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess
import threading

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_PKG_DIR, "csrc")
_LIB_DIR = os.path.join(_PKG_DIR, "lib")
LIB_PATH = os.path.join(_LIB_DIR, "libsplash_b200.so")

SOURCES = (
    "splash_fwd_sm100.cu",
    "splash_fwd_wide_sm100.cu",
    "splash_bwd_sm100.cu",
    "splash_bwd_wide_sm100.cu",
    "splash_host.cu",
    "schedule_builder.cc",
    "maskinfo_builder.cc",
    "segment_schedule.cu",
    "dynamic_schedule.cu",
    "ring_merge.cu",
    "exchange.cu",
    "splash_xla_ffi.cc",  # handlers compile only where xla/ffi/api/ffi.h is on the include path
)

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
)


class SplashError(RuntimeError):
  """A C-ABI call returned a non-zero status."""

  def __init__(self, status: int, what: str):
    self.status = status
    super().__init__(f"{what}: status {status} ({status_str(status)})")


# --------------------------------------------------------------------------------------------
# struct mirrors
# --------------------------------------------------------------------------------------------
class SplashTensor(C.Structure):
  _fields_ = [
      ("data", C.c_void_p),
      ("dtype", C.c_int32),
      ("size", C.c_int64 * 4),
      ("stride", C.c_int64 * 4),
  ]


class SplashMaskFn(C.Structure):
  _fields_ = [
      ("kind", C.c_int32),
      ("offset", C.c_int32),
      ("left", C.c_int32),
      ("right", C.c_int32),
      ("has_left", C.c_int32),
      ("has_right", C.c_int32),
      ("chunk", C.c_int32),
  ]


class SplashMaskNode(C.Structure):
  _fields_ = [
      ("kind", C.c_int32),
      ("left_child", C.c_int32),
      ("right_child", C.c_int32),
      ("fn", SplashMaskFn),
      ("dense", C.c_void_p),
  ]


class SplashMaskInfoOut(C.Structure):
  _fields_ = [
      ("mask_next", C.POINTER(C.c_int32)),
      ("active_rows", C.POINTER(C.c_int32)),
      ("active_cols", C.POINTER(C.c_int32)),
      ("block_mask", C.POINTER(C.c_int32)),
      ("num_active_blocks", C.POINTER(C.c_int32)),
      ("partial_mask_blocks", C.POINTER(C.c_int8)),
      ("n_entries", C.c_int64),
      ("n_shards", C.c_int32),
      ("n_partial", C.c_int32),
      ("all_full", C.c_int32),
  ]


class SplashScheduleOut(C.Structure):
  _fields_ = [
      ("row_ptr", C.POINTER(C.c_int32)),
      ("entries", C.POINTER(C.c_int32)),
      ("n_rows", C.c_int32),
      ("n_entries", C.c_int64),
      ("row_order", C.POINTER(C.c_int32)),
  ]


class SplashDeviceSchedule(C.Structure):
  _fields_ = [
      ("row_ptr", C.c_void_p),
      ("entries", C.c_void_p),
      ("n_rows", C.c_int32),
      ("partial_mask_blocks", C.c_void_p),
      ("block_q", C.c_int32),
      ("block_kv", C.c_int32),
      ("n_entries", C.c_int64),
      ("row_end", C.c_void_p),
      ("entries_per_batch", C.c_int64),
      ("row_order", C.c_void_p),
  ]


class SplashPeerOutput(C.Structure):
  _fields_ = [
      ("ptrs", C.c_void_p),
      ("base_bytes", C.c_int64),
      ("rows_per_peer", C.c_int64),
      ("stride_b", C.c_int64),
      ("stride_h", C.c_int64),
      ("stride_s", C.c_int64),
      ("head0", C.c_int32),
  ]


class SplashFwdArgs(C.Structure):
  _fields_ = [
      ("q", SplashTensor), ("k", SplashTensor), ("v", SplashTensor), ("o", SplashTensor),
      ("logsumexp", C.c_void_p),
      ("max_logits", C.c_void_p),
      ("q_segment_ids", C.c_void_p),
      ("kv_segment_ids", C.c_void_p),
      ("q_sequence", C.c_void_p),
      ("sched", SplashDeviceSchedule),
      ("mask_fn", SplashMaskFn),
      ("scale", C.c_float),
      ("mask_value", C.c_float),
      ("error_record", C.c_void_p),
      ("sinks", C.c_void_p),
      ("max_logit_value", C.c_void_p),
      ("soft_cap", C.c_float),
      ("o_peer", SplashPeerOutput),
  ]


class SplashFwdFp8Args(C.Structure):
  _fields_ = [
      ("base", SplashFwdArgs),
      ("q_scale", C.c_void_p),
      ("k_scale", C.c_void_p),
      ("v_scale", C.c_void_p),
      ("flags", C.c_uint32),
  ]


class SplashBwdArgs(C.Structure):
  _fields_ = [
      ("q", SplashTensor), ("k", SplashTensor), ("v", SplashTensor), ("o", SplashTensor),
      ("d_o", SplashTensor),
      ("dq", SplashTensor), ("dk", SplashTensor), ("dv", SplashTensor),
      ("logsumexp", C.c_void_p),
      ("q_segment_ids", C.c_void_p),
      ("kv_segment_ids", C.c_void_p),
      ("q_sequence", C.c_void_p),
      ("sched_dq", SplashDeviceSchedule),
      ("sched_dkv", SplashDeviceSchedule),
      ("mask_fn", SplashMaskFn),
      ("scale", C.c_float),
      ("workspace", C.c_void_p),
      ("workspace_bytes", C.c_size_t),
      ("error_record", C.c_void_p),
      ("launch_mask", C.c_uint32),
      ("soft_cap", C.c_float),
      ("flags", C.c_uint32),
      ("dq_peer", SplashPeerOutput),
      ("dk_peer", SplashPeerOutput),
      ("dv_peer", SplashPeerOutput),
  ]


BWD_FUSED_DQ = 1  # SplashBwdFlags.SPLASH_BWD_FUSED_DQ
FP8_P_F16 = 1  # SplashFwdFp8Flags.SPLASH_FP8_P_F16


class SplashExchangeArgs(C.Structure):
  _fields_ = [
      ("src", C.c_void_p),
      ("dst_ptrs", C.c_void_p),
      ("world", C.c_int32), ("rank", C.c_int32),
      ("seq_to_head", C.c_int32),
      ("batch", C.c_int64), ("h_loc", C.c_int64), ("s_loc", C.c_int64), ("row_bytes", C.c_int64),
      ("dst_base_bytes", C.c_int64),
  ]


# name -> (restype, argtypes); every function include/splash_b200.h declares.
_PROTOTYPES = {
    "splash_maskinfo_build": (C.c_int, [C.POINTER(SplashMaskNode), C.c_int32, C.c_int64, C.c_int64,
                                        C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_int32, C.POINTER(SplashMaskInfoOut)]),
    "splash_maskinfo_free": (None, [C.POINTER(SplashMaskInfoOut)]),
    "splash_schedule_build": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_int32, C.c_int32, C.POINTER(SplashScheduleOut)]),
    "splash_schedule_free": (None, [C.POINTER(SplashScheduleOut)]),
    "splash_segment_schedule_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int64]),
    "splash_segment_schedule": (C.c_int, [C.POINTER(SplashDeviceSchedule), C.c_int32, C.c_void_p, C.c_void_p,
                                          C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t,
                                          C.POINTER(SplashDeviceSchedule), C.c_void_p]),
    "splash_mask_tile_states": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "splash_dynamic_schedule_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int32, C.c_int64]),
    "splash_dynamic_schedule": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int64, C.c_void_p,
                                          C.c_void_p, C.c_size_t, C.POINTER(SplashDeviceSchedule), C.c_void_p]),
    "splash_fwd": (C.c_int, [C.POINTER(SplashFwdArgs), C.c_void_p]),
    "splash_fwd_fp8": (C.c_int, [C.POINTER(SplashFwdFp8Args), C.c_void_p]),
    "splash_ring_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "splash_bwd_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "splash_bwd_fused_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "splash_bwd": (C.c_int, [C.POINTER(SplashBwdArgs), C.c_void_p]),
    "splash_bwd_static_scratch": (C.c_int, [C.POINTER(SplashBwdArgs), C.c_void_p]),
    "splash_exchange_push": (C.c_int, [C.POINTER(SplashExchangeArgs), C.c_void_p]),
    "splash_read_error": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint32 * 4)]),
    "splash_probe_bounded_wait": (C.c_int, [C.c_void_p, C.c_int64, C.c_uint32, C.c_void_p]),
    "splash_xla_ffi_compiled": (C.c_int, []),
    "splash_xla_ffi_signature": (C.c_char_p, [C.c_int]),
    "splash_status_str": (C.c_char_p, [C.c_int]),
    "splash_version": (C.c_char_p, []),
}

_lib = None
_lock = threading.Lock()


def build(force: bool = False, verbose: bool = False) -> str:
  """Compiles the CUDA/C++ sources into ``lib/libsplash_b200.so`` (sm_100a). Returns its path."""
  srcs = [os.path.join(_CSRC, s) for s in SOURCES if os.path.exists(os.path.join(_CSRC, s))]
  deps = srcs + [os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith(".cuh")]
  deps.append(os.path.join(os.path.dirname(_PKG_DIR), "include", "splash_b200.h"))
  if not force and os.path.exists(LIB_PATH):
    newest = max(os.path.getmtime(d) for d in deps)
    if os.path.getmtime(LIB_PATH) >= newest:
      return LIB_PATH
  os.makedirs(_LIB_DIR, exist_ok=True)
  nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
  cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH, *srcs]
  if verbose:
    cmd.insert(1, "-Xptxas")
    cmd.insert(2, "-v")
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
  if verbose:
    print(res.stderr)
  return LIB_PATH


def lib() -> C.CDLL:
  """Loads the library (building it first if absent). Raises if that is impossible."""
  global _lib
  with _lock:
    if _lib is None:
      if not os.path.exists(LIB_PATH):
        build()
      handle = C.CDLL(LIB_PATH)
      for name, (restype, argtypes) in _PROTOTYPES.items():
        fn = getattr(handle, name)  # AttributeError if the symbol is missing
        fn.restype = restype
        fn.argtypes = argtypes
      _lib = handle
    return _lib


def exported_symbols() -> tuple[str, ...]:
  return tuple(_PROTOTYPES)


def status_str(status: int) -> str:
  try:
    return lib().splash_status_str(int(status)).decode()
  except Exception:  # pylint: disable=broad-except
    return "?"


def check(status: int, what: str) -> None:
  if status != 0:
    raise SplashError(int(status), what)
