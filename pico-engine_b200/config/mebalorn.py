"""Typed configuration of the Mebalorn decoder, read from its own config.json keys.

The design: an embedding with a sinusoidal position vector added; layers that each name their mixer
(``"attention"``: grouped softmax attention without positions in the scores, with query/key norm, a sink
in the softmax denominator and mixing of the heads' weights; ``"mingru"``: a gated recurrence) and an
optional dense feed-forward; both halves of a layer read the same residual stream through a layer norm
and a short causal convolution that is added to its input; a final layer norm, the head, and a soft cap
on the logits.  Every size and every constant that may differ between models comes from config.json:

    {"architecture": "Mebalorn", "vocab": V, "width": W, "norm": {"eps": e}, "canon": {"taps": k},
     "logit_softcap": c, "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim",
     "scale"}, "mlp": {"kind": "dense", "ff": F} | null}, {"type": "mingru", "mixer": {"width"}, ...}]}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import register_architecture
from .specs import (CausalConvAddSpec, ConfigError, DenseMLPSpec, HeadMixAttentionSpec, LayerNormSpec, LayerSpec,
                    MinGRUSpec, ModelPlan, NoPositionSpec, ScheduleEntry, SinusoidAddSpec)

# Positions are float32 in the position vector's angles: every integer below 2^24 is exact there.
MAX_POSITIONS = 1 << 24
SINUSOID_BASE = 10000.0


def _int(d: dict, key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}{key} must be a positive integer, found {v!r}")
    return v


def _number(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f"{where}{key} must be a positive number, found {v!r}")
    return float(v)


@dataclass(frozen=True)
class MebalornLayer:
    """One entry of ``layers``.  ``kind`` "attention" uses heads .. scale, "mingru" uses ``state_width``;
    ``ff`` None: the layer has no feed-forward."""
    kind: str
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 0.0
    state_width: int = 0
    ff: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict, i: int) -> "MebalornLayer":
        where = f"layers[{i}]."
        if not isinstance(d, dict) or "type" not in d:
            raise ConfigError(f"layers[{i}] needs a type")
        kind, m, mlp = d["type"], d.get("mixer"), d.get("mlp")
        if not isinstance(m, dict):
            raise ConfigError(f"{where}mixer must be an object with the mixer's sizes")
        ff = None
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"{where}mlp.kind must be \"dense\" (or mlp null), found {mlp!r}")
            ff = _int(mlp, "ff", where + "mlp.")
        if kind == "attention":
            layer = cls(kind, heads=_int(m, "heads", where + "mixer."), kv_heads=_int(m, "kv_heads", where + "mixer."),
                        dim=_int(m, "dim", where + "mixer."), vdim=_int(m, "vdim", where + "mixer."),
                        scale=_number(m, "scale", where + "mixer."), ff=ff)
            if layer.heads % layer.kv_heads:
                raise ConfigError(f"{where}mixer: {layer.heads} heads cannot share {layer.kv_heads} key/value heads evenly")
            return layer
        if kind == "mingru":
            return cls(kind, state_width=_int(m, "width", where + "mixer."), ff=ff)
        raise ConfigError(f"{where}type must be \"attention\" or \"mingru\", found {kind!r}")

    def to_dict(self) -> dict:
        mlp = None if self.ff is None else {"ff": self.ff, "kind": "dense"}
        if self.kind == "attention":
            mixer = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        else:
            mixer = {"width": self.state_width}
        return {"mixer": mixer, "mlp": mlp, "type": self.kind}


@dataclass(frozen=True)
class MebalornConfig:
    ARCHITECTURE = "Mebalorn"

    vocab: int
    width: int
    layers: Tuple[MebalornLayer, ...]
    norm_eps: float
    canon_taps: int
    logit_softcap: Optional[float] = None

    @classmethod
    def from_dict(cls, d: dict) -> "MebalornConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "canon") if d.get(k) is None]
        if missing:
            raise ConfigError("config.json lacks " + ", ".join(missing))
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("layers must be a non-empty list")
        if not isinstance(d["norm"], dict) or not isinstance(d["canon"], dict):
            raise ConfigError("norm and canon must be objects ({\"eps\": ...}, {\"taps\": ...})")
        cap = d.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
            raise ConfigError(f"logit_softcap must be a positive number or absent, found {cap!r}")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                   layers=tuple(MebalornLayer.from_dict(x, i) for i, x in enumerate(d["layers"])),
                   norm_eps=_number(d["norm"], "eps", "norm."), canon_taps=_int(d["canon"], "taps", "canon."),
                   logit_softcap=float(cap) if cap else None)

    def to_dict(self) -> dict:
        d = {"architecture": self.ARCHITECTURE, "canon": {"taps": self.canon_taps},
             "layers": [x.to_dict() for x in self.layers], "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
             "width": self.width}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d

    # ---------------------------------------------------------------- the plan

    def plan(self) -> ModelPlan:
        W, eps = self.width, self.norm_eps
        layers = []
        for i, x in enumerate(self.layers):
            p = f"l{i}."
            if x.kind == "attention":
                mixer = HeadMixAttentionSpec(
                    hidden=W, n_heads=x.heads, n_kv_heads=x.kv_heads, head_dim=x.dim, v_head_dim=x.vdim, qkv_bias=True,
                    window=None, scale=x.scale, position=NoPositionSpec(), prefix=p + "mix.", norm_eps=eps,
                    q_norm=p + "mix.q.norm", k_norm=p + "mix.k.norm", sink=p + "mix.sink", head_mix=p + "mix.talk")
            else:
                mixer = MinGRUSpec(hidden=W, width=x.state_width, prefix=p + "mix.")
            has_ff = x.ff is not None
            layers.append(LayerSpec(
                mixer=mixer,
                mixer_norm=LayerNormSpec(W, eps, p + "norm1", p + "norm1.b"),
                mixer_input=CausalConvAddSpec(W, self.canon_taps, p + "canon1"),
                feed_forward=DenseMLPSpec(W, x.ff, p + "mlp.", activation="relu2") if has_ff else None,
                feed_forward_norm=LayerNormSpec(W, eps, p + "norm2", p + "norm2.b") if has_ff else None,
                feed_forward_input=CausalConvAddSpec(W, self.canon_taps, p + "canon2") if has_ff else None,
                arrangement="parallel"))
        # A layer without a feed-forward still stores the tensors of its second norm and convolution.
        unused = tuple(f"l{i}.{n}" for i, x in enumerate(self.layers) if x.ff is None
                       for n in ("norm2", "norm2.b", "canon2"))
        plan = ModelPlan(
            architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, embedding="embed",
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            final_norm=LayerNormSpec(W, eps, "final.norm", "final.norm.b"), head="head",
            max_positions=MAX_POSITIONS, ignorable_tensors=unused,
            embedding_position=SinusoidAddSpec(W, SINUSOID_BASE), logit_softcap=self.logit_softcap)
        plan.validate()
        return plan


register_architecture(MebalornConfig.ARCHITECTURE, MebalornConfig)
