"""Types shared by the splash-attention modules.

Mirrors the public names of the reference's
``tokamax/_src/ops/experimental/tpu/splash_attention/base.py`` (``DEFAULT_MASK_VALUE`` :28-30,
``SegmentIds`` :33-54) with torch tensors in place of ``jax.Array``.
"""

from __future__ import annotations

from typing import Any, Final, NamedTuple

import numpy as np

# Logits of masked positions are replaced by this finite value in the reference (base.py:28-30).
# Here it only reaches user-visible results as the logsumexp / max_logits of rows without work.
DEFAULT_MASK_VALUE: Final[float] = -0.7 * float(np.finfo(np.dtype("float32")).max)


class SegmentIds(NamedTuple):
  """Segment ids of the q and kv sequences.

  Tokens attend to each other only where their ids agree; the segment mask is and-ed with the
  static mask.  ``q`` is ``int32[q_seq_len]`` (or ``[batch, q_seq_len]``), ``kv`` likewise.
  """

  q: Any
  kv: Any
