"""Name -> ``from_module`` table of the quantized linear types (kairos/quant_config.py:24-62).

Only the switched-linear types live in this library; the reference's static single-kernel
competitors (W8A8Linear, W4A16Linear, ...) are benchmarks of other projects' kernels and are
rejected with a clear message.
"""
from __future__ import annotations

from .dynamic_linear import DynamicLinear
from .switch_linear import SwitchLinear


class TensorQuantConfig:
    def __init__(self, q_bit, qtype=None, group_size=-1):
        self.bit = q_bit
        self.qtype = qtype      # 'A' or 'S'
        self.group_size = group_size


class LinearQuantConfig:
    def __init__(self, quant_type):
        if quant_type == 'DynamicLinear':
            self.x = TensorQuantConfig(8, 'S')
            self.w = TensorQuantConfig(4, 'A', group_size=128)
            self.from_module = DynamicLinear.from_module
        elif quant_type == 'SwitchLinear':
            self.x = TensorQuantConfig(8, 'S')
            self.w = TensorQuantConfig(4, 'A', group_size=128)
            self.from_module = SwitchLinear.from_module
        else:
            raise ValueError(f'No Supported Linear Type: {quant_type}. '
                             'This library implements DynamicLinear and SwitchLinear.')
