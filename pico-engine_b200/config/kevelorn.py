"""Typed configuration of the Kevelorn decoder, read from its own config.json keys.

The design: pre-norm layers ``x += m * mixer(norm1(x)); x += m * ff(norm2(x))`` with RMS norms whose weights are
stored around zero.  Each layer names its mixer: ``"lightning"`` (linear attention with a fixed decay per head),
``"gla"`` (linear attention with a learned decay per key channel) or ``"parallel"`` (windowed softmax attention with
neighbour-pair rotation, unit-normed queries and keys and an output gate, beside a lightning mixer; the two outputs
are normed and averaged).  The feed-forward is a gated dense one (tanh gelu), a mixture of gated experts with a
shared expert, or absent.  A run of layers may be repeated with the same weights (``loop``); every pass has a cache
of its own, starts by adding a learned vector to the stream, and every pass but the first adds the embedded tokens
again.  Every size and every constant that may differ between models comes from config.json:

    {"architecture": "Kevelorn", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "lightning", "mixer": {"heads", "dim", "vdim", "decay": [per head]}, "mlp": ...},
                {"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": ...},
                {"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                 "rot": {"base", "dims", "scaling": {"factor"}}}, "right": {lightning sizes}}, "mlp": ...}]}
    mlp: null | {"kind": "dense", "ff": F} | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared": {"ff"}}

The rank of the decay projection of a ``gla`` mixer is not in config.json; it is the first dimension of the stored
tensor ``l<i>.mix.a1`` and is read from the checkpoint's header (``from_dict(..., shapes=...)``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

from .registry import register_architecture
from .specs import (BranchSumSpec, ConfigError, GatedAttentionSpec, GatedMLPSpec, LayerSpec, LinearAttentionSpec,
                    MixtureSpec, ModelPlan, NoPositionSpec, RMSNormSpec, RotaryPairsSpec, ScheduleEntry)

# Positions enter float32 angles: every integer below 2^24 is exact there.
MAX_POSITIONS = 1 << 24
DEFAULT_DECAY_RANK = 16


def _int(d: dict, key: str, where: str) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"{where}{key} must be a positive integer, found {v!r}")
    return v


def _number(d: dict, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f"{where}{key} must be a positive number, found {v!r}")
    return float(v)


def _lightning(m: dict, where: str) -> dict:
    heads = _int(m, "heads", where)
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(a, (int, float)) and not isinstance(a, bool) and a >= 0 for a in decay):
        raise ConfigError(f"{where}decay must list one number (not negative) for each of the {heads} heads, found {decay!r}")
    return {"heads": heads, "dim": _int(m, "dim", where), "vdim": _int(m, "vdim", where), "decay": [float(a) for a in decay]}


def _softmax(m: dict, where: str) -> dict:
    out = {"heads": _int(m, "heads", where), "kv_heads": _int(m, "kv_heads", where), "dim": _int(m, "dim", where),
           "vdim": _int(m, "vdim", where), "scale": _number(m, "scale", where)}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['kv_heads']} key/value heads evenly")
    if m.get("mask") is not None:
        out["mask"] = {"size": _int(m["mask"], "size", where + "mask.")}
    rot = m.get("rot")
    if rot is not None:
        r = {"base": _number(rot, "base", where + "rot."), "dims": _int(rot, "dims", where + "rot.")}
        if r["dims"] % 2 or r["dims"] > out["dim"]:
            raise ConfigError(f"{where}rot.dims must be even and at most dim = {out['dim']}, found {r['dims']}")
        if rot.get("scaling") is not None:
            r["scaling"] = {"factor": _number(rot["scaling"], "factor", where + "rot.scaling.")}
        out["rot"] = r
    return out


def _mlp(mlp, where: str) -> Optional[dict]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where}kind must be \"dense\" or \"moe\" (or mlp null), found {mlp!r}")
    if mlp["kind"] == "dense":
        return {"ff": _int(mlp, "ff", where), "kind": "dense"}
    out = {"expert": {"ff": _int(mlp.get("expert"), "ff", where + "expert.")}, "kind": "moe",
           "router": {"experts": _int(mlp.get("router"), "experts", where + "router."),
                      "top": _int(mlp.get("router"), "top", where + "router.")}}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"{where}router.top = {out['router']['top']} exceeds router.experts = {out['router']['experts']}")
    if mlp.get("shared") is not None:
        out["shared"] = {"ff": _int(mlp["shared"], "ff", where + "shared.")}
    return out


@dataclass(frozen=True)
class KevelornLayer:
    """One entry of ``layers``: ``kind`` and the checked ``mixer`` and ``mlp`` objects as config.json spells them."""
    kind: str
    mixer: dict = field(hash=False)
    mlp: Optional[dict] = field(default=None, hash=False)
    decay_rank: int = DEFAULT_DECAY_RANK              # gla only

    @classmethod
    def from_dict(cls, d: dict, i: int, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "KevelornLayer":
        where = f"layers[{i}]."
        if not isinstance(d, dict) or "type" not in d:
            raise ConfigError(f"layers[{i}] needs a type")
        kind, m = d["type"], d.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"{where}mixer must be an object with the mixer's sizes")
        mlp = _mlp(d.get("mlp"), where + "mlp.")
        if kind == "lightning":
            return cls(kind, _lightning(m, where + "mixer."), mlp)
        if kind == "gla":
            mixer = {"heads": _int(m, "heads", where + "mixer."), "dim": _int(m, "dim", where + "mixer."),
                     "vdim": _int(m, "vdim", where + "mixer."), "tau": _number(m, "tau", where + "mixer.")}
            rank = _int(m, "rank", where + "mixer.") if m.get("rank") is not None else DEFAULT_DECAY_RANK
            stored = (shapes or {}).get(f"l{i}.mix.a1")
            if stored is not None and len(stored) == 2:
                rank = int(stored[0])
            return cls(kind, mixer, mlp, decay_rank=rank)
        if kind == "parallel":
            if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                raise ConfigError(f"{where}mixer needs the objects left and right")
            return cls(kind, {"left": _softmax(m["left"], where + "mixer.left."),
                              "right": _lightning(m["right"], where + "mixer.right.")}, mlp)
        raise ConfigError(f"{where}type must be \"lightning\", \"gla\" or \"parallel\", found {kind!r}")

    def to_dict(self) -> dict:
        mixer = dict(self.mixer)
        if self.kind == "gla" and self.decay_rank != DEFAULT_DECAY_RANK:
            mixer["rank"] = self.decay_rank
        return {"mixer": mixer, "mlp": self.mlp, "type": self.kind}


@dataclass(frozen=True)
class KevelornConfig:
    ARCHITECTURE = "Kevelorn"
    READS_TENSOR_SHAPES = True

    vocab: int
    width: int
    layers: Tuple[KevelornLayer, ...]
    norm_eps: float
    residual_mult: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None       # (start, stop, times)

    @classmethod
    def from_dict(cls, d: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "KevelornConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if d.get(k) is None]
        if missing:
            raise ConfigError("config.json lacks " + ", ".join(missing))
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("layers must be a non-empty list")
        if not isinstance(d["norm"], dict):
            raise ConfigError("norm must be an object ({\"eps\": ...})")
        loop = d.get("loop")
        if loop is not None:
            a, b, n = loop.get("start"), loop.get("stop"), loop.get("times")
            if not all(isinstance(v, int) and not isinstance(v, bool) for v in (a, b, n)) or not 0 <= a < b <= len(d["layers"]) or n < 1:
                raise ConfigError(f"loop needs 0 <= start < stop <= {len(d['layers'])} layers and times >= 1, found {loop!r}")
            loop = (a, b, n)
        mult = d.get("residual_mult", 1.0)
        if isinstance(mult, bool) or not isinstance(mult, (int, float)):
            raise ConfigError(f"residual_mult must be a number, found {mult!r}")
        return cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                   layers=tuple(KevelornLayer.from_dict(x, i, shapes) for i, x in enumerate(d["layers"])),
                   norm_eps=_number(d["norm"], "eps", "norm."), residual_mult=float(mult), loop=loop)

    def to_dict(self) -> dict:
        d = {"architecture": self.ARCHITECTURE, "layers": [x.to_dict() for x in self.layers], "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    # ---------------------------------------------------------------- the plan

    def _lightning_spec(self, m: dict, prefix: str) -> LinearAttentionSpec:
        return LinearAttentionSpec(hidden=self.width, n_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"], prefix=prefix,
                                   head_decay=tuple(m["decay"]), qk_activation="silu", v_activation="silu", norm_over="heads",
                                   norm_eps=self.norm_eps, gate_activation="sigmoid")

    def _mixer_spec(self, x: KevelornLayer, p: str):
        W, eps, m = self.width, self.norm_eps, x.mixer
        if x.kind == "lightning":
            return self._lightning_spec(m, p)
        if x.kind == "gla":
            return LinearAttentionSpec(hidden=W, n_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"], prefix=p,
                                       decay_names=("a1", "a2", "a2.b"), decay_rank=x.decay_rank, decay_tau=m["tau"],
                                       q_scale=m["dim"] ** -0.5, norm_over="head", norm_eps=eps, gate_activation="silu")
        left = m["left"]
        rot = left.get("rot")
        position = NoPositionSpec() if rot is None else RotaryPairsSpec(
            head_dim=left["dim"], dims=rot["dims"], base=rot["base"], factor=(rot.get("scaling") or {}).get("factor", 1.0))
        attention = GatedAttentionSpec(hidden=W, n_heads=left["heads"], n_kv_heads=left["kv_heads"], head_dim=left["dim"],
                                       v_head_dim=left["vdim"], window=(left.get("mask") or {}).get("size"), scale=left["scale"],
                                       position=position, prefix=p + "left.", qk_unit_norm=True, norm_eps=eps)
        return BranchSumSpec(hidden=W, branches=(attention, self._lightning_spec(m["right"], p + "right.")),
                             out_norms=(p + "left.out", p + "right.out"), norm_eps=eps, weight=0.5)

    def _ff_spec(self, mlp: Optional[dict], p: str):
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return GatedMLPSpec(self.width, mlp["ff"], p, activation="gelu_tanh")
        shared = mlp.get("shared")
        return MixtureSpec(hidden=self.width, n_experts=mlp["router"]["experts"], top_k=mlp["router"]["top"],
                           intermediate=mlp["expert"]["ff"], prefix=p, activation="silu",
                           shared_intermediate=None if shared is None else shared["ff"])

    def plan(self) -> ModelPlan:
        W, eps = self.width, self.norm_eps
        layers = []
        for i, x in enumerate(self.layers):
            p = f"l{i}."
            ff = self._ff_spec(x.mlp, p + "mlp.")
            layers.append(LayerSpec(mixer=self._mixer_spec(x, p + "mix."),
                                    mixer_norm=RMSNormSpec(W, eps, p + "norm1", one_plus=True),
                                    feed_forward=ff,
                                    feed_forward_norm=None if ff is None else RMSNormSpec(W, eps, p + "norm2", one_plus=True),
                                    arrangement="pre_norm", residual_scale=self.residual_mult))
        n = len(layers)
        if self.loop is None:
            schedule = [ScheduleEntry(i) for i in range(n)]
        else:
            a, b, times = self.loop
            schedule = [ScheduleEntry(i) for i in range(a)]
            for t in range(times):
                schedule += [ScheduleEntry(i, add_embedding=(i == a and t > 0), add_vector=("loop.step", t) if i == a else None)
                             for i in range(a, b)]
            schedule += [ScheduleEntry(i) for i in range(b, n)]
        # A layer without a feed-forward may still store its second norm.
        unused = tuple(f"l{i}.norm2" for i, x in enumerate(self.layers) if x.mlp is None)
        plan = ModelPlan(architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=W, embedding="embed",
                         layers=tuple(layers), schedule=tuple(schedule),
                         final_norm=RMSNormSpec(W, eps, "final.norm", one_plus=True), head="head",
                         max_positions=MAX_POSITIONS, ignorable_tensors=unused,
                         stream_vectors=(("loop.step", self.loop[2]),) if self.loop is not None else ())
        plan.validate()
        return plan


register_architecture(KevelornConfig.ARCHITECTURE, KevelornConfig)
