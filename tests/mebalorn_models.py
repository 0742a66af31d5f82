"""Small Mebalorn configurations and random weights for the tests, written out independently of the library.

The configurations differ from one another in every size and option: the number and order of layers, heads
per key/value head (1, 2, 3), key and value sizes (equal, larger, smaller), state width against model width,
taps (1 to 5), layers without a feed-forward, with and without a soft cap.  Weights have the scale
1/sqrt(inputs) so that activations keep their size and attention scores spread over several units: weights
of 0.02 would hide a key read from the wrong place behind a nearly uniform softmax.
"""
from __future__ import annotations

import torch


def attention(heads, kv_heads, dim, vdim, scale, ff):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mingru(width, ff):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, taps, eps, cap, layers):
    d = {"architecture": "Mebalorn", "vocab": vocab, "width": width, "canon": {"taps": taps}, "norm": {"eps": eps},
         "layers": layers}
    if cap is not None:
        d["logit_softcap"] = cap
    return d


CONFIGS = {
    # mixed order, 3 query heads a key/value head, values smaller and larger than keys, a layer without feed-forward
    "M1": config(300, 72, 4, 1e-5, 9.0, [attention(6, 2, 32, 16, 0.21, 136), mingru(40, None),
                                         attention(4, 4, 16, 48, 0.3, 64), mingru(96, 200)]),
    # one tap (the convolution keeps no state), no soft cap, one head
    "M2": config(128, 48, 1, 1e-6, None, [mingru(48, 96), attention(1, 1, 64, 64, 0.125, None)]),
    # two taps, attention first and last, two heads on one key/value head, odd sizes
    "M3": config(200, 40, 2, 3e-6, 30.0, [attention(2, 1, 24, 40, 0.2, 56), mingru(24, 72), attention(2, 2, 40, 8, 0.17, 48)]),
    # five taps, recurrence only
    "M4": config(96, 56, 5, 1e-5, 5.0, [mingru(64, 80), mingru(56, None)]),
    # many heads (beyond what the tensor-core kernels take), head sizes that are no multiples of 8, eight taps, a wide state
    "M5": config(150, 100, 8, 1e-6, 12.0, [attention(40, 8, 20, 12, 0.22, 72), mingru(520, 40)]),
    # nine taps (more than the fused norm + convolution kernel takes), key and value sizes 80 and 48, a width that is no multiple of 4
    "M6": config(90, 50, 9, 2e-6, None, [mingru(30, None), attention(6, 3, 80, 48, 0.11, 60)]),
}


def tensor_shapes(cfg: dict) -> dict:
    W, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    shapes = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,), "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes.update({p + "norm1": (W,), p + "norm1.b": (W,), p + "canon1": (W, taps)})
        if layer["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * D, W), p + "mix.q.b": (H * D,), p + "mix.k": (G * D, W), p + "mix.k.b": (G * D,),
                           p + "mix.v": (G * Dv, W), p + "mix.v.b": (G * Dv,), p + "mix.q.norm": (D,), p + "mix.k.norm": (D,),
                           p + "mix.talk": (H, H), p + "mix.sink": (H,), p + "mix.o": (W, H * Dv)})
        else:
            S = m["width"]
            shapes.update({p + "mix.z": (S, W), p + "mix.z.b": (S,), p + "mix.x": (S, W), p + "mix.x.b": (S,),
                           p + "mix.g": (S, W), p + "mix.o": (W, S)})
        if layer["mlp"] is not None:
            F = layer["mlp"]["ff"]
            shapes.update({p + "norm2": (W,), p + "norm2.b": (W,), p + "canon2": (W, taps),
                           p + "mlp.up": (F, W), p + "mlp.down": (W, F)})
    return shapes


def make_weights(cfg: dict, seed: int) -> dict:
    """Random weights rounded to bfloat16 values (kept in float32 here)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name in ("final.norm",) or name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "talk":
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last in ("canon1", "canon2"):
            t = 0.5 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * shape[1] ** -0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def requests_for(cfg: dict, lengths, seed: int = 7) -> dict:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def plain_logits(cfg: dict, weights: dict, requests: dict) -> dict:
    import plain_mebalorn as plain
    out = {}
    for rid, toks in requests.items():
        lg = plain.logits(toks, weights, cfg).numpy()
        for p in range(len(toks)):
            out[(rid, p)] = lg[p]
    return out
