"""The C-ABI library loads and exports every symbol include/splash_b200.h declares (no GPU)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from tokamax_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
  text = open(os.path.join(ROOT, "include", "splash_b200.h")).read()
  text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
  names = re.findall(r"\b(splash_[a-z0-9_]+)\s*\(", text)
  return sorted(set(names))


def test_header_functions_are_all_exported_and_bound():
  declared = _declared_functions()
  assert len(declared) >= 10
  lib = C.CDLL(_native.build())
  for name in declared:
    assert hasattr(lib, name), f"{name} declared in the header but not exported"
  assert sorted(_native.exported_symbols()) == declared


def test_status_strings_and_version():
  lib = _native.lib()
  assert lib.splash_version().decode().startswith("splash_b200")
  for code in range(0, -8, -1):
    text = lib.splash_status_str(code).decode()
    assert text and text != "unknown status"
  assert lib.splash_status_str(-99).decode() == "unknown status"


def test_null_and_invalid_arguments_return_status_codes():
  lib = _native.lib()
  assert lib.splash_fwd(None, None) == -1
  assert lib.splash_bwd(None, None) == -1
  assert lib.splash_fwd_fp8(None, None) == -1
  assert lib.splash_read_error(None, None, None) == -1
  assert lib.splash_bwd_workspace_bytes(0, 1, 1) == 0
  assert lib.splash_bwd_workspace_bytes(2, 8, 1024) == 2 * (2 * 8 * 1024 * 4)  # di and -lse*log2e
  assert lib.splash_bwd_workspace_bytes(1, 1, 33) % 256 == 0
  out = _native.SplashScheduleOut()
  state = np.ones((2, 2), np.int32)
  assert lib.splash_schedule_build(state.ctypes.data, None, 2, 2, 100, 128, 0, C.byref(out)) == -1
  assert lib.splash_schedule_build(state.ctypes.data, None, 2, 2, 128, 128, 7, C.byref(out)) == -1
  assert lib.splash_schedule_build(None, None, 2, 2, 128, 128, 0, C.byref(out)) == -1
  mi = _native.SplashMaskInfoOut()
  node = _native.SplashMaskNode()
  node.kind = 1
  node.fn.kind = 1
  assert lib.splash_maskinfo_build(C.byref(node), 1, 100, 128, 128, 128, 0, 1, 1, 1, C.byref(mi)) == -1
  node.kind = 5  # AND without children
  node.left_child = node.right_child = 3
  assert lib.splash_maskinfo_build(C.byref(node), 1, 128, 128, 128, 128, 0, 1, 1, 1, C.byref(mi)) == -1
  lib.splash_maskinfo_free(C.byref(mi))  # freeing an empty result is harmless


def test_forward_rejects_bad_tensors_before_touching_the_gpu():
  """Argument validation happens on the host, so it can be exercised without a device."""
  lib = _native.lib()
  a = _native.SplashFwdArgs()
  assert lib.splash_fwd(C.byref(a), None) == -1  # null data pointers
  for t in (a.q, a.k, a.v, a.o):
    t.data = 4096
    t.dtype = 0
    for i, s in enumerate((1, 2, 256, 320)):
      t.size[i] = s
    t.stride[0], t.stride[1], t.stride[2], t.stride[3] = 2 * 256 * 320, 256 * 320, 320, 1
  assert lib.splash_fwd(C.byref(a), None) == -2  # head_dim 320: unsupported, not invalid
  for t in (a.q, a.k, a.v, a.o):
    t.size[3] = 60
  assert lib.splash_fwd(C.byref(a), None) == -1  # head_dim 60: rows are not a multiple of 16 bytes
  for t in (a.q, a.k, a.v, a.o):
    t.size[3] = 64  # head dims below 128 are taken; the call now fails later, on the missing tables
  assert lib.splash_fwd(C.byref(a), None) == -1
  a.q.dtype = 1
  assert lib.splash_fwd(C.byref(a), None) == -2  # fp32 inputs
  a.q.dtype = 0
  a.q.stride[2] = 316
  assert lib.splash_fwd(C.byref(a), None) == -1  # row stride not a multiple of 16 bytes


def test_ctypes_structs_have_the_layout_the_c_header_gives_them(tmp_path):
  """sizeof and the offset of the last field of every args struct, as a C compiler sees the header,
  against the ctypes mirrors the Python layer fills."""
  import shutil
  import subprocess

  cc = shutil.which("gcc") or shutil.which("cc")
  if cc is None:
    pytest.skip("needs a C compiler")
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  structs = {
      "SplashTensor": "stride", "SplashMaskFn": None, "SplashDeviceSchedule": "row_order", "SplashPeerOutput": "head0",
      "SplashFwdArgs": "o_peer", "SplashFwdFp8Args": "flags", "SplashBwdArgs": "dv_peer", "SplashExchangeArgs": "dst_base_bytes",
  }
  lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "splash_b200.h"', "int main(void) {"]
  for name, last in structs.items():
    lines.append(f'  printf("{name} %zu %zu\\n", sizeof({name}), ' +
                 (f"offsetof({name}, {last})" if last else "(size_t)0") + ");")
  lines += ["  return 0;", "}"]
  src = tmp_path / "layout.c"
  src.write_text("\n".join(lines))
  exe = tmp_path / "layout"
  subprocess.run([cc, "-std=c99", "-I", os.path.join(root, "include"), str(src), "-o", str(exe)], check=True)
  out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
  seen = 0
  for line in out:
    if not line.strip():
      continue
    name, size, offset = line.split()
    mirror = getattr(_native, name)
    assert C.sizeof(mirror) == int(size), name
    last = structs[name]
    if last:
      assert getattr(mirror, last).offset == int(offset), (name, last)
    seen += 1
  assert seen == len(structs)
