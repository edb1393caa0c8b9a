"""``SwitchLinear``: the all-formats-resident ablation (kairos/switch_linear.py:43-213).

Same dispatch as ``DynamicLinear``, but the int8 and fp16 forms of the weight stay resident, so
a call never pays a conversion.  Here that is the same layer bound to a context whose
conversion cache is unbounded and filled when the module is built.
"""
from __future__ import annotations

import torch

from .dynamic_linear import COMP_TYPE_NAME, DynamicLinear
from .runtime import Context


class SwitchLinear(DynamicLinear):
    prof = None
    context = None
    _resident_ctx = {}

    def _cache_context(self):
        if type(self).context is not None:
            return type(self).context
        dev = self.qweight.device
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        if idx not in SwitchLinear._resident_ctx:
            SwitchLinear._resident_ctx[idx] = Context(torch.device('cuda', idx), cache_bytes=None)
        return SwitchLinear._resident_ctx[idx]

    @classmethod
    @torch.no_grad()
    def from_module(cls, linear, device, return_dtype=torch.float16, init_only=False, name=''):
        q_linear = super().from_module(linear, device, return_dtype, init_only, name)
        if not init_only and q_linear.qweight.is_cuda:
            q_linear.make_resident()
        return q_linear

    @torch.no_grad()
    def make_resident(self):
        """Fill the int8 (smq_weight) and fp16 (ori_weight) forms now."""
        self.prefetch(COMP_TYPE_NAME['w8a8'])
        self.prefetch(COMP_TYPE_NAME['fp16'])

    def init(self):
        super().init()
        if self.qweight.is_cuda:
            self.make_resident()
