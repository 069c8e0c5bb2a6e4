"""Constants of the fp8 recipe (scope parity: reference src/nanotron/fp8/constants.py).

Recipe of this framework: e4m3 for activations and weights in the forward, e5m2 for gradients; activations / gradients scaled
per 1 x 128 block, weights per 128 x 128 block, scales fp32 ``amax / max`` (no history, no delayed scaling: every tensor is
scaled by its own current maximum, which block scaling makes cheap).  The per-tensor, power-of-two scaling of ``fp8/tensor.py``
is kept for interchange with checkpoints and tools that expect one scale per tensor.
"""
from nanotron_b200.fp8.dtypes import DTypes

BLOCK = 128
FP8_MAX = {DTypes.FP8E4M3: 448.0, DTypes.FP8E5M2: 57344.0}
FORWARD_DTYPE = DTypes.FP8E4M3
GRADIENT_DTYPE = DTypes.FP8E5M2
FP8_DTYPES = (DTypes.FP8E4M3, DTypes.FP8E5M2)
# per-tensor scaling: head-room (in powers of two) left below the format's maximum, and how often the scale is refreshed
DEFAULT_MARGIN = 0
DEFAULT_INTERVAL = 1
