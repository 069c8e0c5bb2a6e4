from nanotron_b200.fp8.linear import FP8Linear  # noqa: F401
from nanotron_b200.fp8.quantize import FP8BlockTensor, dequantize, quantize_1x128, quantize_128x128  # noqa: F401
