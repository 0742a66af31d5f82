"""Small Kevelorn configurations and random weights for the tests, written out independently of the library.

The configurations differ from one another in every size and option: the order of the mixers, heads per key/value
head (1, 2, 3), key and value sizes (equal, larger, smaller, multiples of 16 or not), windows below and above a cache
page and none at all, rotation of all or some entries with and without stretched positions, decays of 1 and far below,
ranks of the decay projection, experts with top 1, top = experts and in between, with and without a shared expert,
layers without a feed-forward, loops that start at the first layer, run once, or are absent, residual factors
including 1, and norm constants from 2e-6 to 3e-3 (a large one shows where it is added; it also keeps the norm of a
mixer's output from blowing up rounding noise where that output is nearly zero, at a sequence's first tokens).  Weights have the scale 1/sqrt(inputs) so that activations keep their size and scores spread.
"""
from __future__ import annotations

import torch


def lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def gla(heads, dim, vdim, tau, mlp):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def parallel(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right["mixer"]}, "mlp": mlp}


def softmax(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        d["mask"] = {"size": window}
    if rot is not None:
        dims, base, factor = rot
        d["rot"] = {"dims": dims, "base": base}
        if factor is not None:
            d["rot"]["scaling"] = {"factor": factor}
    return d


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        d["shared"] = {"ff": shared}
    return d


def config(vocab, width, eps, mult, layers, loop=None):
    d = {"architecture": "Kevelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if loop is not None:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


RANKS = {"K1": 8, "K2": 5, "K3": 16, "K4": 3}

CONFIGS = {
    # the loop starts at the first layer and runs three times; 3 query heads a key/value head; part of a head is rotated,
    # positions stretched; a window shorter than a page; experts 5 / top 2 with a larger shared expert; a layer without feed-forward
    "K1": config(300, 72, 1e-5, 0.5, [
        parallel(softmax(6, 2, 32, 32, 0.4, window=40, rot=(16, 10000.0, 4.0)), lightning(2, 16, 24, [0.9, 0.5], None), moe(5, 2, 24, 40)),
        gla(3, 24, 16, 8.0, dense(100)),
        lightning(3, 40, 8, [0.97, 0.8, 0.3], None)], loop=(0, 2, 3)),
    # no loop, residual factor 1; values larger than keys (the kernels for unequal sizes); every entry rotated, positions
    # not stretched; a window of one page and a bit; top 1 of 3 experts without a shared one; one head
    "K2": config(128, 48, 1e-2, 1.0, [
        gla(1, 32, 48, 2.0, moe(3, 1, 32)),
        parallel(softmax(4, 4, 16, 40, 0.5, window=70, rot=(16, 500.0, None)), lightning(1, 16, 8, [1.0], None), dense(64)),
        lightning(2, 64, 32, [1.0, 0.99], dense(40))]),
    # a loop of one pass in the middle; head size 64 (the tensor-memory prompt kernel); no window; no rotation; top = experts
    "K3": config(200, 64, 1e-3, 0.3, [
        lightning(2, 32, 32, [0.6, 0.95], dense(96)),
        parallel(softmax(2, 1, 64, 64, 0.3), lightning(4, 16, 16, [0.99, 0.9, 0.7, 0.2], None), moe(2, 2, 48, 16)),
        gla(2, 16, 32, 16.0, None)], loop=(1, 2, 1)),
    # odd sizes: a width that is no multiple of 4, head sizes 24 (no multiple of 16), 136 (more than 128) and 12; a window of 2;
    # the loop ends with the last layer; 7 experts top 3
    "K4": config(90, 50, 2e-6, 0.7, [
        gla(2, 136, 12, 4.0, dense(36)),
        parallel(softmax(3, 1, 24, 24, 0.35, window=2, rot=(24, 100.0, 2.0)), lightning(3, 20, 12, [0.5, 0.9, 0.999], None), moe(7, 3, 20, 12))],
        loop=(1, 2, 2)),
}


def tensor_shapes(cfg: dict, rank: int) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("loop"):
        shapes["loop.step"] = (cfg["loop"]["times"], W)

    def linear_attention(p, m):
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        shapes.update({p + "q": (H * D, W), p + "k": (H * D, W), p + "v": (H * Dv, W), p + "g": (H * Dv, W), p + "o": (W, H * Dv)})
        return H, D, Dv

    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "lightning":
            H, D, Dv = linear_attention(p + "mix.", m)
            shapes[p + "mix.norm"] = (H * Dv,)
        elif layer["type"] == "gla":
            H, D, Dv = linear_attention(p + "mix.", m)
            shapes.update({p + "mix.norm": (Dv,), p + "mix.a1": (rank, W), p + "mix.a2": (H * D, rank), p + "mix.a2.b": (H * D,)})
        else:
            a = m["left"]
            H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            shapes.update({q + "q": (H * D, W), q + "k": (G * D, W), q + "v": (G * Dv, W), q + "g": (H * Dv, W), q + "o": (W, H * Dv),
                           q + "out": (W,), p + "mix.right.out": (W,)})
            H, D, Dv = linear_attention(p + "mix.right.", m["right"])
            shapes[p + "mix.right.norm"] = (H * Dv,)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        shapes[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            experts = [(f"{p}mlp.e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                experts.append((p + "mlp.shared.", mlp["shared"]["ff"]))
                shapes[p + "mlp.shared.sg"] = (1, W)
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for q, F in experts:
                shapes.update({q + "gate": (F, W), q + "up": (F, W), q + "down": (W, F)})
    return shapes


def make_weights(cfg: dict, seed: int, rank: int) -> dict:
    """Random weights rounded to bfloat16 values (kept in float32 here)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            t = 0.1 * torch.randn(shape, generator=g)                 # stored around zero
        elif last in ("norm", "out"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name == "loop.step":
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 1.0 + torch.randn(shape, generator=g)                 # decay logits spread around sigmoid(1)
        elif last == "router" or last == "sg":
            t = torch.randn(shape, generator=g) * 4.0 * shape[1] ** -0.5   # logits a few units apart: no close calls
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * shape[1] ** -0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def requests_for(cfg: dict, lengths, seed: int = 7) -> dict:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


_cache = {}
CLOSE_CALL = 0.08       # router logits of the tests spread over several units; bfloat16 rounding moves them by a hundredth or two


def plain_logits(cfg: dict, weights: dict, requests: dict, close_calls: set | None = None) -> dict:
    """{(request, position): logits row} of the plain implementation in float64 (kept: the tests ask for the same
    requests in several ways of cutting).  ``close_calls`` receives the (request, position) pairs at which some router
    of the plain run chose its last expert by less than CLOSE_CALL: there a run in bfloat16 may rightly choose another
    expert, and the comparison in bfloat16 leaves those places out (float32 runs are compared everywhere)."""
    import plain_kevelorn as plain
    out = {}
    w64 = None
    for rid, toks in requests.items():
        key = (id(weights), tuple(toks))
        if key not in _cache:
            if w64 is None:
                w64 = {n: t.double() for n, t in weights.items()}
            plain.ROUTER_GAPS = []
            logits = plain.logits(toks, w64, cfg).float().numpy()
            gaps, plain.ROUTER_GAPS = plain.ROUTER_GAPS, None
            close = torch.stack(gaps).min(0).values < CLOSE_CALL if gaps else torch.zeros(len(toks), dtype=torch.bool)
            _cache[key] = (logits, close.tolist())
        logits, close = _cache[key]
        for p in range(len(toks)):
            out[(rid, p)] = logits[p]
            if close_calls is not None and close[p]:
                close_calls.add((rid, p))
    return out
