"""kairos_b200: B200-native switched quantized linear (DynamicLinear / SwitchLinear).

Importing the package loads libkairos_b200.so; there is no fallback when it is missing.
"""
from ._lib import KairosError, LIB_PATH, lib  # noqa: F401
from .dynamic_linear import COMP_TYPE_ID, COMP_TYPE_NAME, DynamicLinear  # noqa: F401
from .perf_profiler import LUT, Profiler  # noqa: F401
from .quant_config import LinearQuantConfig  # noqa: F401
from .quant_model import quantize_model  # noqa: F401
from .switch_linear import SwitchLinear  # noqa: F401

__all__ = ['DynamicLinear', 'SwitchLinear', 'Profiler', 'LUT', 'LinearQuantConfig', 'quantize_model',
           'COMP_TYPE_NAME', 'COMP_TYPE_ID', 'KairosError']
