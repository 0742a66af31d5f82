"""A plain, slow implementation of the Kevelorn decoder: whole sequences, no cache, no batching,
one function per mechanism, written out from the design's equations.  It shares no code with the
library and is the oracle of the GPU tests.

Notation.  A sequence has tokens at positions p = 0 .. n-1; ``x`` is the residual stream [n, width].
``cfg`` is the parsed config.json, ``w`` maps tensor names to tensors; matrices are [out, in] and applied
as W x.  Everything runs in the dtype of ``x`` (the tests use float64).
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces

def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, weight, eps):
    """The norm in front of a sublayer and before the head: its weight is stored around zero."""
    return rms_unit(x, eps) * (1 + weight)


def norm_plain(x, weight, eps):
    return rms_unit(x, eps) * weight


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def lin(w, h):
    return h @ w.T


# ------------------------------------------------------------------ rotation

def rotate_pairs(u, first, dims, base, factor):
    """u [n, heads, D]: neighbours (2i, 2i+1) of the first ``dims`` entries of every head are turned by the angle
    p * base^(-2i/dims) / factor, p = first + row; the rest of a head stays."""
    out = u.clone()
    n = u.shape[0]
    for t in range(n):
        p = first + t
        for i in range(dims // 2):
            a = p * (base ** (-2.0 * i / dims)) / factor
            c, s = math.cos(a), math.sin(a)
            a0, a1 = u[t, :, 2 * i], u[t, :, 2 * i + 1]
            out[t, :, 2 * i] = a0 * c - a1 * s
            out[t, :, 2 * i + 1] = a1 * c + a0 * s
    return out


# ------------------------------------------------------------------ mixers

def window_attention(q, k, v, scale, window):
    """q [n, H, D], k [n, G, D], v [n, G, Dv] -> [n, H, Dv]; query i sees keys j with 0 <= i - j < window
    (all earlier keys if window is None); query head h reads key/value head h // (H / G)."""
    n, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    out = torch.zeros(n, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        c = h // per
        for i in range(n):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo: i + 1, c] @ q[i, h]) * scale
            e = torch.exp(s - s.max())
            out[i, h] = (e / e.sum()) @ v[lo: i + 1, c]
    return out


def linear_recurrence(q, k, v, decay, state=None):
    """Per head S_t = diag(decay_t) S_(t-1) + k_t v_t^T and o_t = S_t^T q_t.  q, k [n, H, D], v [n, H, Dv];
    ``decay`` [n, H, D] (a decay per key channel; a decay per head is the same number on all its channels).
    Returns o [n, H, Dv] and the last state [H, D, Dv]."""
    n, H, D = q.shape
    Dv = v.shape[2]
    S = torch.zeros(H, D, Dv, dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros(n, H, Dv, dtype=q.dtype)
    for t in range(n):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


def mixer_softmax(h, w, p, m, eps, first=0):
    """The softmax-attention mixer: interleaved rotation of q and k, unit RMS norm of every head, window, sigmoid
    output gate.  ``m`` holds heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor}}, mask {size}."""
    n = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(w[p + "q"], h).view(n, H, D)
    k = lin(w[p + "k"], h).view(n, G, D)
    v = lin(w[p + "v"], h).view(n, G, Dv)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = rotate_pairs(q, first, rot["dims"], rot["base"], factor)
        k = rotate_pairs(k, first, rot["dims"], rot["base"], factor)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    window = (m.get("mask") or {}).get("size")
    o = window_attention(q, k, v, m["scale"], window).reshape(n, H * Dv)
    return lin(w[p + "o"], o * sigmoid(lin(w[p + "g"], h)))


def mixer_lightning(h, w, p, m, eps):
    """Linear attention with a fixed decay per head: silu on q, k, v; all heads normed together; sigmoid gate."""
    n = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(lin(w[p + "q"], h)).view(n, H, D)
    k = silu(lin(w[p + "k"], h)).view(n, H, D)
    v = silu(lin(w[p + "v"], h)).view(n, H, Dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype).view(1, H, 1).expand(n, H, D)
    o, _ = linear_recurrence(q, k, v, decay)
    o = norm_plain(o.reshape(n, H * Dv), w[p + "norm"], eps)
    return lin(w[p + "o"], o * sigmoid(lin(w[p + "g"], h)))


def mixer_gla(h, w, p, m, eps):
    """Linear attention with a learned decay per key channel: alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau); queries
    scaled by dim^(-1/2); every head normed by itself over vdim with one shared weight; silu gate."""
    n = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (lin(w[p + "q"], h) * D ** -0.5).view(n, H, D)
    k = lin(w[p + "k"], h).view(n, H, D)
    v = lin(w[p + "v"], h).view(n, H, Dv)
    z = lin(w[p + "a2"], lin(w[p + "a1"], h)) + w[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).view(n, H, D)
    o, _ = linear_recurrence(q, k, v, alpha)
    o = norm_plain(o, w[p + "norm"], eps).reshape(n, H * Dv)
    return lin(w[p + "o"], o * silu(lin(w[p + "g"], h)))


def mixer_parallel(h, w, p, m, eps):
    """Softmax attention and fixed-decay linear attention side by side on the same input; each output is normed
    over the model width with a plain weight, and the result is half their sum."""
    left = mixer_softmax(h, w, p + "left.", m["left"], eps)
    right = mixer_lightning(h, w, p + "right.", m["right"], eps)
    return 0.5 * (norm_plain(left, w[p + "left.out"], eps) + norm_plain(right, w[p + "right.out"], eps))


# ------------------------------------------------------------------ feed-forwards

def gated_mlp(h, w, p, act):
    return lin(w[p + "down"], act(lin(w[p + "gate"], h)) * lin(w[p + "up"], h))


ROUTER_GAPS = None      # a list: every call of ``mixture`` appends, per token, how far the last chosen logit lies above the next one


def mixture(h, w, p, mlp):
    """Every token takes its ``top`` experts with the largest router logits, weighted by the softmax over those
    logits alone; a shared expert, scaled by one sigmoid gate a token, is added."""
    n = h.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = lin(w[p + "router"], h)
    if ROUTER_GAPS is not None and top < E:
        ordered = z.sort(-1, descending=True).values
        ROUTER_GAPS.append(ordered[:, top - 1] - ordered[:, top])
    out = torch.zeros(n, w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(n):
        order = sorted(range(E), key=lambda e: -float(z[t, e]))[:top]
        zt = torch.stack([z[t, e] for e in order])
        wt = torch.exp(zt - zt.max())
        wt = wt / wt.sum()
        for j, e in enumerate(order):
            out[t] += wt[j] * gated_mlp(h[t: t + 1], w, f"{p}e{e}.", silu)[0]
    if mlp.get("shared"):
        out = out + gated_mlp(h, w, p + "shared.", silu) * sigmoid(lin(w[p + "shared.sg"], h))
    return out


# ------------------------------------------------------------------ the model

def run_layer(x, w, i, layer, cfg):
    eps, mult, p = cfg["norm"]["eps"], cfg["residual_mult"], f"l{i}."
    h = norm_one_plus(x, w[p + "norm1"], eps)
    mixer = {"parallel": mixer_parallel, "lightning": mixer_lightning, "gla": mixer_gla}[layer["type"]]
    x = x + mult * mixer(h, w, p + "mix.", layer["mixer"], eps)
    mlp = layer.get("mlp")
    if mlp:
        h = norm_one_plus(x, w[p + "norm2"], eps)
        ff = gated_mlp(h, w, p + "mlp.", gelu_tanh) if mlp["kind"] == "dense" else mixture(h, w, p + "mlp.", mlp)
        x = x + mult * ff
    return x


def layer_runs(cfg):
    """The order in which layers run: (layer, number of the pass if it is the first layer of a pass, else None)."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def hidden(tokens, w, cfg, trace=None):
    """The residual stream after the last layer; ``trace`` (a list) receives it after every layer run."""
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x = run_layer(x, w, i, cfg["layers"][i], cfg)
        if trace is not None:
            trace.append(x.clone())
    return x


def logits(tokens, w, cfg):
    """[n, vocab] for one sequence."""
    x = hidden(tokens, w, cfg)
    return lin(w["head"], norm_one_plus(x, w["final.norm"], cfg["norm"]["eps"]))


def generate(tokens, w, cfg, n_new):
    """Greedy continuation: recomputes the whole sequence for every new token."""
    tokens = list(tokens)
    for _ in range(n_new):
        tokens.append(int(torch.argmax(logits(tokens, w, cfg)[-1])))
    return tokens
