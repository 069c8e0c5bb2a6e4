from nanotron_b200.fp8.dtypes import DTypes  # noqa: F401
from nanotron_b200.fp8.linear import FP8Linear  # noqa: F401
from nanotron_b200.fp8.meta import FP8Meta  # noqa: F401
from nanotron_b200.fp8.parameter import FP8Parameter, QuantizedWeightCache, weight_cache  # noqa: F401
from nanotron_b200.fp8.quantize import FP8BlockTensor, dequantize, quantize_1x128, quantize_128x128  # noqa: F401
from nanotron_b200.fp8.tensor import FP8Tensor, convert_tensor_from_fp8  # noqa: F401
