"""The minGRU mixer: a gated recurrence whose gates read only the current token."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds
from ..config.specs import MinGRUSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import Mixer, register_mixer


@register_mixer(MinGRUSpec)
class MinGRU(Mixer):
    """z = sigmoid(W_z h + b_z), c = g(W_x h + b_x) with g(u) = u + 1/2 for u >= 0 and sigmoid(u) below,
    S_t = (1 - z) S_(t-1) + z c, output W_o (S_t * silu(W_g h)).  The three input projections are one product
    on concatenated weights; gates, candidate and state are float32, the state is a row of the cache's state
    area, zero for a new sequence.  All it reads of the step lies on the device, so a decode step with this
    mixer can be a captured graph."""

    def __init__(self, spec: MinGRUSpec, dtype, device):
        super().__init__(spec, dtype, device)
        self.w_in = self.b_in = self.w_o = None

    def _names(self):
        s = self.spec
        return [s.prefix + n for n in (s.z_name, s.x_name, s.g_name, s.o_name)]

    def expected_tensors(self):
        s = self.spec
        z, x, g, o = self._names()
        return {z: ParamSpec((s.width, s.hidden)), z + s.bias_suffix: ParamSpec((s.width,)),
                x: ParamSpec((s.width, s.hidden)), x + s.bias_suffix: ParamSpec((s.width,)),
                g: ParamSpec((s.width, s.hidden)), o: ParamSpec((s.hidden, s.width))}

    def take_tensors(self, get):
        s = self.spec
        z, x, g, o = self._names()
        self.w_in = torch.cat([get(z), get(x), get(g)], dim=0).contiguous()
        bz, bx = get(z + s.bias_suffix), get(x + s.bias_suffix)
        self.b_in = torch.cat([bz, bx, torch.zeros_like(bz)]).contiguous()          # the gate projection has no bias
        self.w_o = get(o)

    def cache_needs(self):
        return CacheNeeds(kv=None, state_elems=self.spec.width)

    def gated_state(self, h, ctx, cache_entry):
        """S_t * silu(g_t) [T, width] of the step's tokens; the sequences' states move on."""
        proj = linear(h, self.w_in, self.b_in, out_dtype=ctx.dtype)
        # sequences that bring many tokens: a scan over chunks; a step of (about) one token each: token after token
        return kernels.mingru(proj, ctx.state(cache_entry), 0, ctx.tok_row, ctx.row_first, ctx.row_lens, ctx.slots,
                              chunked=ctx.T > 2 * ctx.B)

    def apply(self, h, ctx, entry, cache_entry, owns_cache):
        return linear(self.gated_state(h, ctx, cache_entry), self.w_o, out_dtype=ctx.dtype)

    def add_output_to(self, x, h, ctx, entry, cache_entry, owns_cache) -> None:
        """x += mixer(h) for rows h that are normed (and filtered) already."""
        linear(self.gated_state(h, ctx, cache_entry), self.w_o, accumulate_into=x)
