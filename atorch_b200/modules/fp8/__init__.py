from .precision_switchable_linear import PrecisionSwitchableLinear
from .quantize import (ScaleType, block_quantize, dequantize, scaled_gemm, tile_quantize,
                       tile_quantize_transposed)
from .quantized_grouped_linear import ATorchGroupedLinear
from .scaled_linear import ScaledLinear
from .utils import (convert_linears_to_fp8, get_fp8_module_count, get_fp8_quantize_underflows,
                    set_linear_modules_precision)
