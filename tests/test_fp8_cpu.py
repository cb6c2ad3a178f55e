"""Host side of the e4m3 path: block-scaled quantisation round trip (no GPU)."""
import torch

from tokamax_b200 import fp8


def test_quantize_dequantize_round_trip():
  g = torch.Generator().manual_seed(5)
  x = torch.randn(2, 3, 384, 128, generator=g).to(torch.bfloat16)
  x[0, 1, 128:256] = 0  # an all-zero tile gets scale 0 and decodes to zeros
  x[1, 2, 256:] *= 100.0
  t = fp8.quantize_e4m3(x)
  assert t.data.dtype == torch.float8_e4m3fn and t.data.shape == x.shape
  assert t.scale.dtype == torch.float32 and t.scale.shape == (2, 3, 3)
  amax = x.float().reshape(2, 3, 3, -1).abs().amax(-1)
  assert torch.equal(t.scale, amax / 448.0)
  assert t.scale[0, 1, 1] == 0
  y = fp8.dequantize_e4m3(t, torch.float32)
  assert torch.count_nonzero(y[0, 1, 128:256]) == 0
  # e4m3 keeps 3 mantissa bits: error <= 2^-4 relative for normal values, and at most half the
  # smallest subnormal step (2^-10 of the scaled range) otherwise
  bound = x.float().abs() * 2.0**-4 + (t.scale * 2.0**-10).repeat_interleave(128, dim=2)[..., None]
  assert ((y - x.float()).abs() <= bound).all()
  # the largest value of every tile is kept exactly
  assert torch.allclose(y.reshape(2, 3, 3, -1).abs().amax(-1), amax, rtol=1e-6)


def test_quantize_rejects_ragged_sequence():
  import pytest
  with pytest.raises(ValueError):
    fp8.quantize_e4m3(torch.zeros(1, 1, 100, 128))
