"""Positions that are added to the embedded stream."""
from __future__ import annotations

import torch

from ..config.specs import SinusoidAddSpec
from ..ops import kernels
from .base import StreamPosition, register_stream_position


@register_stream_position(SinusoidAddSpec)
class SinusoidAdd(StreamPosition):
    """x[t, 2i] += sin(p_t * base^(-2i/size)), x[t, 2i + 1] += cos of the same angle.  The frequencies are
    computed once on the host in float64 and rounded to float32, so that they do not depend on the device's
    ``pow``; the angle is their float32 product with the position."""

    def __init__(self, spec: SinusoidAddSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.freq = None

    def prepare(self, max_positions: int) -> None:
        if self.freq is None:
            i = torch.arange((self.spec.size + 1) // 2, dtype=torch.float64)
            self.freq = torch.pow(torch.tensor(self.spec.base, dtype=torch.float64), -2.0 * i / self.spec.size) \
                .to(torch.float32).to(self.device).contiguous()

    def weights(self):
        return []

    def add_to(self, x, ctx) -> None:
        kernels.add_sinusoid(x, ctx.tok_pos, self.freq)
