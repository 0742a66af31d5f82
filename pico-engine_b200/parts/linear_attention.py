"""Linear attention: a recurrence over a matrix state per head, with a fixed decay per head or a learned one per key channel."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds
from ..config.specs import ConfigError, LinearAttentionSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import Mixer, first_product, last_product_into, normed_rows, register_mixer


@register_mixer(LinearAttentionSpec)
class LinearAttention(Mixer):
    """S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head; o normed (over all heads together or head by head),
    multiplied by a gate of the mixer's input, projected by W_o.  q, k, v and the gate are one product on concatenated
    weights; activations of q, k, v, the decay (from its logits), the state, the output, its norm and the gate are float32
    in either dtype (csrc/linear_attention.cu, csrc/gated_ops.cu).  The state [heads, head_dim, v_head_dim] is a run of
    the layer's row of the cache's state area, starting at ``state_offset`` (a mixer that holds several mixers places
    them one behind the other).  All it reads of the step lies on the device, so a decode step can be a captured graph."""

    takes_out_dtype = True      # apply(..., out_dtype=) gives the product's float32 sums where the caller goes on in float32

    def __init__(self, spec: LinearAttentionSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if (spec.head_decay is None) == (spec.decay_names is None):
            raise ConfigError("linear attention needs either a decay per head or the names of a decay projection")
        if spec.head_decay is not None and len(spec.head_decay) != spec.n_heads:
            raise ConfigError(f"{len(spec.head_decay)} decays for {spec.n_heads} heads")
        if spec.head_dim > 256:
            raise ConfigError(f"head size {spec.head_dim} is not taken: the recurrence kernel takes up to 256")
        if spec.norm_over not in ("heads", "head"):
            raise ConfigError(f"norm_over must be \"heads\" or \"head\", not {spec.norm_over!r}")
        for a in (spec.qk_activation, spec.v_activation):
            if a not in kernels.LA_ACTIVATIONS:
                raise ConfigError(f"activation {a!r} is not known; known: {', '.join(sorted(kernels.LA_ACTIVATIONS))}")
        if spec.gate_activation not in kernels.GATE_ACTIVATIONS:
            raise ConfigError(f"gate activation {spec.gate_activation!r} is not known")
        self.state_offset = 0
        self.w_in = self.w_o = self.norm = self.head_decay = self.w_a1 = self.w_a2 = self.b_a2 = None

    def _sizes(self):
        s = self.spec
        return s.n_heads * s.head_dim, s.n_heads * s.v_head_dim

    def expected_tensors(self):
        s = self.spec
        qk, vo = self._sizes()
        p = s.prefix
        out = {p + s.q_name: ParamSpec((qk, s.hidden)), p + s.k_name: ParamSpec((qk, s.hidden)),
               p + s.v_name: ParamSpec((vo, s.hidden)), p + s.g_name: ParamSpec((vo, s.hidden)),
               p + s.o_name: ParamSpec((s.hidden, vo)),
               p + s.norm_name: ParamSpec((vo if s.norm_over == "heads" else s.v_head_dim,), init="one_plus_normal")}
        if s.decay_names is not None:
            a1, a2, b = s.decay_names
            out.update({p + a1: ParamSpec((s.decay_rank, s.hidden)), p + a2: ParamSpec((qk, s.decay_rank)), p + b: ParamSpec((qk,))})
        return out

    def take_tensors(self, get):
        s, p = self.spec, self.spec.prefix
        self.w_in = torch.cat([get(p + n) for n in (s.q_name, s.k_name, s.v_name, s.g_name)], dim=0).contiguous()
        self.w_o = get(p + s.o_name)
        self.norm = get(p + s.norm_name)
        if s.decay_names is not None:
            a1, a2, b = s.decay_names
            self.w_a1, self.w_a2, self.b_a2 = get(p + a1), get(p + a2), get(p + b)
        else:
            self.head_decay = torch.tensor(s.head_decay, dtype=torch.float32, device=self.device)

    def prepare(self, max_positions):
        from ..ops.library import gated
        gated()                                            # build or load this part's kernels now, loudly

    def cache_needs(self):
        s = self.spec
        return CacheNeeds(kv=None, state_elems=s.n_heads * s.head_dim * s.v_head_dim)

    def gated_output(self, h, ctx, cache_entry, x_norm=None):
        """norm(o_t) * gate [T, heads * v_head_dim] of the step's tokens; the sequences' states move on.  The input is
        either normed rows ``h`` or ``x_norm`` = (stream, its norm)."""
        s = self.spec
        qk, vo = self._sizes()
        rows = normed_rows(h, x_norm, ctx, self.w_in)
        proj = first_product(*rows, self.w_in, ctx)
        logits = None
        if self.w_a1 is not None:
            if rows[0] is None and not kernels.fused_takes(proj.shape[0], self.w_a1, rows[1]):
                rows = (x_norm[1].forward(x_norm[0], ctx.dtype), None, None, 0.0)
            logits = linear(first_product(*rows, self.w_a1, ctx), self.w_a2, self.b_a2, out_dtype=torch.float32)
        # Token after token, a block a (sequence, head, 32 columns of the state), unless that leaves the GPU empty: few sequences
        # with many tokens run as three passes over chunks.  Measured on a B200 (16 heads of 128 x 128): one prompt of 2,048
        # tokens 319 us in chunks against 709 us, four such prompts 1,985 us against 1,062 us.  (Either way gives the same
        # numbers up to float32 rounding; rows that bring a few tokens, such as the idle rows of a padded step, do not count.)
        long_rows = sum(1 for n in ctx.lens if n > 64)
        blocks = long_rows * s.n_heads * ((s.v_head_dim + 31) // 32)
        o = kernels.linear_attention(proj, 0, qk, 2 * qk, s.n_heads, s.head_dim, s.v_head_dim, ctx.state(cache_entry),
                                     self.state_offset, ctx.row_first, ctx.row_lens, ctx.slots,
                                     chunked=0 < blocks < 192,
                                     head_decay=self.head_decay, decay_logits=logits, inv_tau=1.0 / s.decay_tau,
                                     q_scale=s.q_scale, qk_activation=s.qk_activation, v_activation=s.v_activation)
        return kernels.gated_norm(o, vo if s.norm_over == "heads" else s.v_head_dim, self.norm, s.norm_eps, proj, 2 * qk + vo,
                                  s.gate_activation, ctx.dtype)

    def apply(self, h, ctx, entry, cache_entry, owns_cache, out_dtype=None, x_norm=None):
        return linear(self.gated_output(h, ctx, cache_entry, x_norm), self.w_o, out_dtype=out_dtype or ctx.dtype)

    def add_normed_to(self, x, norm, scale, ctx, entry, cache_entry, owns_cache) -> bool:
        """x += scale * mixer(norm(x)), the norm in the first product and the sum in the last where they take the sizes."""
        last_product_into(x, self.gated_output(None, ctx, cache_entry, (x, norm)), self.w_o, scale, ctx)
        return True
