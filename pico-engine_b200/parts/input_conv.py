"""The short causal convolution that is added to what a sublayer reads."""
from __future__ import annotations

import torch

from ..config.specs import CausalConvAddSpec, ConfigError
from ..ops import kernels
from ..weights.loader import ParamSpec
from .base import InputFilter, register_input_filter


@register_input_filter(CausalConvAddSpec)
class CausalConvAdd(InputFilter):
    """o_t = y_t + sum_j c[:, j] * y_(t - taps + 1 + j) per channel, zeros before a sequence's start.  The last
    taps - 1 rows y of a sequence are its state (float32, newest first), so that a step continues where the
    last one ended whatever the cut."""

    def __init__(self, spec: CausalConvAddSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.taps < 1:
            raise ConfigError(f"a convolution needs at least one tap, not {spec.taps}")
        self.taps_weight = None

    def expected_tensors(self):
        return {self.spec.weight: ParamSpec((self.spec.size, self.spec.taps))}

    def take_tensors(self, get):
        self.taps_weight = get(self.spec.weight)

    def state_elems(self) -> int:
        return (self.spec.taps - 1) * self.spec.size

    def apply(self, y, ctx, state, offset, out_dtype):
        return kernels.causal_conv_add(y, self.taps_weight, state, offset, ctx.tok_row, ctx.row_first, ctx.row_lens,
                                       ctx.slots, out_dtype)
