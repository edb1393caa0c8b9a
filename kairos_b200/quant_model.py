"""Swap every ``nn.Linear`` inside a model's decoder layers for a switched linear
(kairos/quant_model.py:8-56): same functions, same returned per-layer ``{name: type}`` list.
The strategy is an argument (the reference reads it from stdin at import time)."""
from __future__ import annotations

import gc

import torch

from .quant_config import LinearQuantConfig


@torch.no_grad()
def get_name_linears(module):
    return {name: m for name, m in module.named_modules() if isinstance(m, torch.nn.Linear)}


@torch.no_grad()
def set_op_by_name(layer, name, new_module):
    levels = name.split('.')
    mod = layer
    for lv in levels[:-1]:
        mod = mod[int(lv)] if lv.isdigit() else getattr(mod, lv)
    setattr(mod, levels[-1], new_module)


@torch.no_grad()
def quantize_model(model, init_only=False, _quant_config=None, quant_strategy='DynamicLinear', device=None):
    """Replace the linears of ``model.model.layers`` in place; lm_head stays fp16.
    Returns the per-layer list of {linear name: quant type}."""
    quant_config = []
    layers = model.model.layers
    for layer_idx in range(len(layers)):
        quant_config.append({})
        layer = layers[layer_idx]
        for name, module in get_name_linears(layer).items():
            if _quant_config is not None:
                quant_type = _quant_config[layer_idx][name]
            else:
                quant_type = quant_strategy
            quant_config[layer_idx][name] = quant_type
            dev = device if device is not None else module.weight.device
            q_linear = LinearQuantConfig(quant_type).from_module(module, dev, init_only=init_only)
            if not init_only:
                module.cpu()
            set_op_by_name(layer, name, q_linear)
        gc.collect()
    return quant_config
