"""Several mixers side by side on one input, their normed outputs summed."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds
from ..config.specs import BranchSumSpec, ConfigError
from ..ops import kernels
from ..weights.loader import ParamSpec
from .base import MIXERS, Mixer, build_part, register_mixer


@register_mixer(BranchSumSpec)
class BranchSum(Mixer):
    """weight * sum_i rmsnorm(branch_i(h)) * w_i.  The branches are ordinary mixers; at most one of them keeps keys and
    values (they share the layer's cache entry), and their states lie one behind the other in the layer's row of the
    state area (each branch is told its ``state_offset``).  The norms of the branches' outputs, their sum and the
    sum into the residual stream are one float32 kernel (csrc/gated_ops.cu)."""

    def __init__(self, spec: BranchSumSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if not 1 <= len(spec.branches) <= 4 or len(spec.out_norms) != len(spec.branches):
            raise ConfigError("a sum of branches takes one to four branches and a norm weight for each")
        self.branches = [build_part(MIXERS, "mixer", b, dtype, device) for b in spec.branches]
        needs = [b.cache_needs() for b in self.branches]
        if sum(1 for n in needs if n.kv is not None) > 1:
            raise ConfigError("only one branch of a sum may keep keys and values")
        if any(n.state_elems and n.state_dtype != "float32" for n in needs):
            raise ConfigError("branches keep float32 state")
        offset = 0
        for b, n in zip(self.branches, needs):
            if n.state_elems and not hasattr(b, "state_offset"):
                raise ConfigError(f"{type(b).__name__} keeps state but cannot be placed behind another part's (no state_offset)")
            if hasattr(b, "state_offset"):
                b.state_offset = offset
            offset += n.state_elems
        self._needs = CacheNeeds(kv=next((n.kv for n in needs if n.kv is not None), None), state_elems=offset)
        self.out_norms = None

    def expected_tensors(self):
        out = {}
        for b in self.branches:
            out.update(b.expected_tensors())
        out.update({n: ParamSpec((self.spec.hidden,), init="one_plus_normal") for n in self.spec.out_norms})
        return out

    def take_tensors(self, get):
        for b in self.branches:
            b.take_tensors(get)
        self.out_norms = [get(n) for n in self.spec.out_norms]

    def prepare(self, max_positions):
        for b in self.branches:
            b.prepare(max_positions)

    def weights(self):
        return [t for b in self.branches for t in b.weights()] + list(self.out_norms or [])

    def cache_needs(self):
        return self._needs

    def add_normed_to(self, x, norm, scale, ctx, entry, cache_entry, owns_cache) -> bool:
        """x += scale * mixer(norm(x)); branches that can take the norm into their first product."""
        if not all(getattr(b, "takes_out_dtype", False) for b in self.branches):
            return False
        outs = [b.apply(None, ctx, entry, cache_entry, owns_cache, out_dtype=x.dtype, x_norm=(x, norm)) for b in self.branches]
        kernels.normed_sum_add(x, outs, self.out_norms, self.spec.norm_eps, scale * self.spec.weight)
        return True

    def add_scaled_to(self, x, h, scale, ctx, entry, cache_entry, owns_cache) -> None:
        """x += scale * mixer(h) for normed rows h."""
        outs = [b.apply(h, ctx, entry, cache_entry, owns_cache, **({"out_dtype": x.dtype} if getattr(b, "takes_out_dtype", False) else {}))
                for b in self.branches]
        if len({o.dtype for o in outs}) > 1:
            outs = [o.float() for o in outs]
        kernels.normed_sum_add(x, outs, self.out_norms, self.spec.norm_eps, scale * self.spec.weight)

    def apply(self, h, ctx, entry, cache_entry, owns_cache):
        y = torch.zeros(h.shape[0], self.spec.hidden, dtype=torch.float32, device=h.device)
        self.add_scaled_to(y, h, 1.0, ctx, entry, cache_entry, owns_cache)
        return y
