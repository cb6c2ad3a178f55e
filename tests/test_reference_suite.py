"""Runs the reference's own mask / MaskInfo test-suite against this package's modules.

Only possible where a checkout of the reference is present (SPLASH_REFERENCE_ROOT points at it);
skipped elsewhere — the committed golden tables (test_maskinfo_golden.py) carry the same pin to other machines.
The suite is the reference's splash_attention_mask_test.py (126 tests, literal expected tables
at :752-1750), with its ``mask_lib`` / ``mask_info_lib`` aliases pointed at tokamax_b200.
"""
import subprocess
import sys
import os

import pytest

from oracle import ref_loader

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_SCRIPT = """
import sys
sys.path.insert(0, {root!r})
from oracle import ref_loader
import tokamax_b200.splash_attention_mask as mm
import tokamax_b200.splash_attention_mask_info as mi
r = ref_loader.run_reference_mask_tests(mm, mi)
print("RESULT", r.testsRun, len(r.failures), len(r.errors))
for t, tb in r.failures + r.errors:
  print("BAD", t.id())
"""


@pytest.mark.skipif(not ref_loader.available(), reason="SPLASH_REFERENCE_ROOT is not set to a checkout of the reference")
def test_reference_mask_suite_passes_on_this_implementation():
  # a fresh interpreter: the stub jax module and the aliased test module stay out of this process
  out = subprocess.run([sys.executable, "-c", _SCRIPT.format(root=ROOT)], capture_output=True, text=True,
                       timeout=600)
  line = [l for l in out.stdout.splitlines() if l.startswith("RESULT")]
  assert line, out.stdout + out.stderr
  run, failures, errors = map(int, line[0].split()[1:])
  assert run >= 120 and failures == 0 and errors == 0, out.stdout
