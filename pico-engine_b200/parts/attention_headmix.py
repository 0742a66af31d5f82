"""Grouped softmax attention whose weights are mixed across heads, with query/key norm and a sink."""
from __future__ import annotations

import torch

from ..cache import CacheNeeds, KVNeed
from ..config.specs import ConfigError, HeadMixAttentionSpec, NoPositionSpec
from ..ops import kernels, linear
from ..weights.loader import ParamSpec
from .base import Mixer, register_mixer


@register_mixer(HeadMixAttentionSpec)
class HeadMixAttention(Mixer):
    """One product for q, k and v (with biases), RMS norm of every query and key head, keys and values into the
    cache, then attention in which every head's softmax (whose denominator also holds exp(sink_h)) is mixed
    with the other heads' by ``head_mix`` before it meets the values of the head's own key/value head, then
    the output projection.  Keys and values may have different head sizes.  Scores, weights and the mixing are
    float32 in either dtype (csrc/attention_headmix.cu)."""

    def __init__(self, spec: HeadMixAttentionSpec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.n_heads % spec.n_kv_heads:
            raise ConfigError(f"{spec.n_heads} query heads cannot share {spec.n_kv_heads} key/value heads evenly")
        if not isinstance(spec.position, NoPositionSpec):
            raise ConfigError("attention with mixed heads takes queries and keys as projected (no position encoding)")
        if spec.n_heads * spec.v_head_dim > 16384:
            raise ConfigError(f"{spec.n_heads} heads of value size {spec.v_head_dim} are not taken: their product may be "
                              f"16384 at most")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError(f"window {spec.window} must be positive")
        self.w_qkv = self.b_qkv = self.w_o = self.q_norm = self.k_norm = self.sink = self.head_mix = None

    def _names(self):
        s = self.spec
        return [s.prefix + n for n in (s.q_name, s.k_name, s.v_name, s.o_name)]

    def expected_tensors(self):
        s = self.spec
        q, k, v, o = self._names()
        out = {q: ParamSpec((s.n_heads * s.head_dim, s.hidden)), k: ParamSpec((s.n_kv_heads * s.head_dim, s.hidden)),
               v: ParamSpec((s.n_kv_heads * s.v_head_dim, s.hidden)), o: ParamSpec((s.hidden, s.n_heads * s.v_head_dim))}
        if s.qkv_bias:
            out.update({q + s.bias_suffix: ParamSpec((s.n_heads * s.head_dim,)),
                        k + s.bias_suffix: ParamSpec((s.n_kv_heads * s.head_dim,)),
                        v + s.bias_suffix: ParamSpec((s.n_kv_heads * s.v_head_dim,))})
        for name in (s.q_norm, s.k_norm):
            if name is not None:
                out[name] = ParamSpec((s.head_dim,), init="one_plus_normal")
        if s.sink is not None:
            out[s.sink] = ParamSpec((s.n_heads,))
        if s.head_mix is not None:
            out[s.head_mix] = ParamSpec((s.n_heads, s.n_heads), init="identity_plus_normal")
        return out

    def take_tensors(self, get):
        s = self.spec
        q, k, v, o = self._names()
        self.w_qkv = torch.cat([get(q), get(k), get(v)], dim=0).contiguous()
        if s.qkv_bias:
            self.b_qkv = torch.cat([get(n + s.bias_suffix) for n in (q, k, v)]).contiguous()
        self.w_o = get(o)
        self.q_norm = None if s.q_norm is None else get(s.q_norm)
        self.k_norm = None if s.k_norm is None else get(s.k_norm)
        # the sink and the mixing matrix enter float32 arithmetic: kept in float32 whatever they were stored in
        self.sink = None if s.sink is None else get(s.sink).float().contiguous()
        self.head_mix = None if s.head_mix is None else get(s.head_mix).float().contiguous()

    def cache_needs(self):
        s = self.spec
        return CacheNeeds(kv=KVNeed(s.n_kv_heads, s.head_dim, s.window,
                                    v_head_dim=None if s.v_head_dim == s.head_dim else s.v_head_dim))

    def attend(self, h, ctx, cache_entry, owns_cache):
        """The heads' outputs [T, n_heads * v_head_dim] for normed rows h."""
        s = self.spec
        kv = ctx.kv(cache_entry)
        qkv = linear(h, self.w_qkv, self.b_qkv, out_dtype=ctx.dtype)
        store = owns_cache
        kernels.qknorm_store(qkv, s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim, self.q_norm, self.k_norm, s.norm_eps,
                             ctx.tok_pos, ctx.tok_row, kv.k if store else None, kv.v if store else None,
                             kv.table if store else None, kv.stride)
        return kernels.attention_headmix(qkv, qkv.shape[1], s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim, kv.k, kv.v,
                                         kv.table, kv.stride, ctx.tok_pos, ctx.tok_row, s.window, s.scale, self.sink,
                                         self.head_mix, ctx)

    def apply(self, h, ctx, entry, cache_entry, owns_cache):
        return linear(self.attend(h, ctx, cache_entry, owns_cache), self.w_o, out_dtype=ctx.dtype)

    def add_output_to(self, x, h, ctx, entry, cache_entry, owns_cache) -> None:
        """x += mixer(h) for rows h that are normed (and filtered) already."""
        linear(self.attend(h, ctx, cache_entry, owns_cache), self.w_o, accumulate_into=x)
