"""A plain, slow implementation of the Mebalorn decoder: whole sequences, no cache, no batching,
one function per mechanism, written out from the design's equations.  It shares no code with the
library and is the oracle of the GPU tests.

Notation.  A sequence has tokens at positions p = 0 .. n-1; ``x`` is the residual stream [n, width].
``cfg`` is the parsed config.json, ``w`` maps tensor names to tensors [out, in] (applied as W x).
Everything runs in the dtype of ``x`` (the tests use float64 or float32).
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces

def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * weight + bias, var = mean of squared deviations."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(-1, keepdim=True)
    return d / torch.sqrt(var + eps) * weight + bias


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight, over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def sinusoid(n, width, dtype, first=0, base=10000.0):
    """[n, width]: entry 2i of position p is sin(p * base^(-2i/width)), entry 2i+1 its cosine."""
    out = torch.zeros(n, width, dtype=dtype)
    for p in range(n):
        for i in range((width + 1) // 2):
            a = (first + p) * base ** (-2.0 * i / width)
            out[p, 2 * i] = math.sin(a)
            if 2 * i + 1 < width:
                out[p, 2 * i + 1] = math.cos(a)
    return out


def input_conv(h, taps_weight):
    """h + conv(h) with conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before position 0.
    ``taps_weight`` is [width, taps]."""
    n, width = h.shape
    taps = taps_weight.shape[1]
    out = h.clone()
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] = out[t] + taps_weight[:, j] * h[s]
    return out


# ------------------------------------------------------------------ mixers

def mixed_attention(q, k, v, scale, sink=None, talk=None, window=None):
    """q [n, H, D], k [n, G, D], v [n, G, Dv] of one sequence -> [n, H, Dv].  Causal scores scale * q.k, a softmax
    whose denominator also holds exp(sink_g), the heads' weights mixed by ``talk`` [H, H], each head's mixed weights
    applied to the values of its own key/value head.  ``window`` w: query i sees keys i - w + 1 .. i."""
    n, H, _ = q.shape
    G, Dv = k.shape[1], v.shape[2]
    per = H // G
    weights = torch.zeros(H, n, n, dtype=q.dtype)          # weights[g, i, j], zero for unseen j
    for g in range(H):
        c = g // per
        for i in range(n):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo: i + 1, c] @ q[i, g]) * scale
            top = float(s.max()) if sink is None else max(float(s.max()), float(sink[g]))
            e = torch.exp(s - top)
            den = e.sum() + (0.0 if sink is None else math.exp(float(sink[g]) - top))
            weights[g, i, lo: i + 1] = e / den
    mixed = weights if talk is None else torch.einsum("hg,gij->hij", talk, weights)
    out = torch.zeros(n, H, Dv, dtype=q.dtype)
    for hd in range(H):
        out[:, hd] = mixed[hd] @ v[:, hd // per]
    return out


def attention_mixer(h, w, prefix, m, eps):
    """Projections with biases, RMS norm of every query and key head (one weight vector for all heads), the
    attention above, the output projection.  ``m`` is the layer's mixer dictionary of config.json."""
    n = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(n, H, D)
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(n, G, D)
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(n, G, Dv)
    q = rms_norm(q, w[prefix + "q.norm"], eps)
    k = rms_norm(k, w[prefix + "k.norm"], eps)
    out = mixed_attention(q, k, v, m["scale"], w[prefix + "sink"], w[prefix + "talk"])
    return out.reshape(n, H * Dv) @ w[prefix + "o"].T


def mingru_candidate(u):
    """u + 1/2 where u >= 0, sigmoid(u) where u < 0."""
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru_recurrence(pz, pu, pg, S0=None):
    """Rows of pre-activations [n, W] -> (S_t * silu(pg_t) for every t, the last S)."""
    z = torch.sigmoid(pz)
    c = mingru_candidate(pu)
    gate = pg * torch.sigmoid(pg)
    S = torch.zeros(pz.shape[1], dtype=pz.dtype) if S0 is None else S0
    rows = []
    for t in range(pz.shape[0]):
        S = (1 - z[t]) * S + z[t] * c[t]
        rows.append(S * gate[t])
    return torch.stack(rows), S


def mingru_mixer(h, w, prefix):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t from S = 0; output W_o (S_t * silu(W_g h_t))."""
    y, _ = mingru_recurrence(h @ w[prefix + "z"].T + w[prefix + "z.b"], h @ w[prefix + "x"].T + w[prefix + "x.b"],
                             h @ w[prefix + "g"].T)
    return y @ w[prefix + "o"].T


# ------------------------------------------------------------------ feed-forward

def feed_forward(h, w, prefix):
    """W_down relu(W_up h)^2."""
    a = torch.relu(h @ w[prefix + "up"].T)
    return (a * a) @ w[prefix + "down"].T


# ------------------------------------------------------------------ the model

def layer(x, w, i, spec, cfg):
    """x + mixer(conv(norm1 x)) + ff(conv(norm2 x)), both branches reading the same x."""
    p = f"l{i}."
    eps = cfg["norm"]["eps"]
    h1 = input_conv(layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps), w[p + "canon1"])
    if spec["type"] == "attention":
        y = attention_mixer(h1, w, p + "mix.", spec["mixer"], eps)
    elif spec["type"] == "mingru":
        y = mingru_mixer(h1, w, p + "mix.")
    else:
        raise ValueError(spec["type"])
    if spec.get("mlp") is not None:
        h2 = input_conv(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w[p + "canon2"])
        y = y + feed_forward(h2, w, p + "mlp.")
    return x + y


def hidden_states(tokens, w, cfg, dtype=torch.float64):
    """The residual stream after the embedding and after every layer: list of [n, width]."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    n, width = len(tokens), cfg["width"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] + sinusoid(n, width, dtype)
    out = [x]
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, cfg)
        out.append(x)
    return out, w


def logits(tokens, w, cfg, dtype=torch.float64):
    """[n, vocab]: the final norm, the head and the soft cap cap * tanh(l / cap)."""
    states, w = hidden_states(tokens, w, cfg, dtype)
    h = layer_norm(states[-1], w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"])
    lg = h @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(lg / cap) if cap else lg


def generate(prompt, n_new, w, cfg, dtype=torch.float64):
    """Greedy continuation, recomputing the whole sequence for every token."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(logits(toks, w, cfg, dtype)[-1])))
    return toks[len(prompt):]
