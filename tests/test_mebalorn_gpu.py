"""Mebalorn on the GPU against the plain implementation: each mechanism's kernel alone on inputs that show a fault,
and the whole model through the library's step function, cache, scheduler and entry points, in both dtypes, for
every way of cutting requests into steps."""
from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_mebalorn as plain
import replay
from conftest import write_model
from mebalorn_models import CONFIGS, make_weights, plain_logits, requests_for

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CASES = [(n, d) for n in sorted(CONFIGS) for d in ("float32", "bfloat16")]
LENGTHS = {"M1": [1, 2, 3, 37, 70, 131, 64, 5], "M2": [65, 1, 130, 9, 33, 2], "M3": [3, 129, 31, 32, 64, 1, 200], "M4": [4, 1, 90, 17, 5],
           "M5": [70, 2, 11, 33], "M6": [12, 1, 66, 9, 40]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{(config, dtype): (engine, cfg, weights, folder)}."""
    from pico_engine.engine.engine import Engine
    root = tmp_path_factory.mktemp("mebalorn")
    out = {}
    for k, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        weights = make_weights(cfg, 20 + k)
        folder = write_model(root / name, cfg, weights)
        for dtype in DTYPES:
            out[(name, dtype)] = (Engine(folder, dtype=dtype), cfg, weights, folder)
    return out


def check(models, name, dtype, steps, reqs, what):
    eng, cfg, w, _ = models[(name, dtype)]
    replay.compare(replay.run_in_process(eng, steps), plain_logits(cfg, w, reqs), dtype, what)


# ------------------------------------------------------------------ the whole model, every way of cutting

@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_and_first_tokens(models, name, dtype):
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 1)
    check(models, name, dtype, replay.whole(reqs), reqs, "whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(models, name, dtype):
    """Every request again with its last tokens one at a time (the shortest ones entirely), 100 for the long one."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 2)
    check(models, name, dtype, replay.tail(reqs, 100), reqs, "tail")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompts_in_portions(models, name, dtype):
    """Portions of unequal sizes, then portions of two and three tokens and single tokens in turn: every portion
    starts inside its sequence with the convolutions' and the recurrence's state of the portion before."""
    cfg = CONFIGS[name]
    reqs = requests_for(cfg, LENGTHS[name], 3)
    check(models, name, dtype, replay.pieces(reqs), reqs, "pieces")
    small = requests_for(cfg, [23, 11, 70], 4)
    plan = {}
    for i, (r, toks) in enumerate(small.items()):
        cuts, left, k = [], len(toks), i
        while left:
            c = min(left, (2, 3, 1, 2, 5)[k % 5])
            cuts.append(c); left -= c; k += 1
        plan[r] = (i, cuts)
    check(models, name, dtype, replay.scheduled(small, plan), small, "small portions")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("batch_size,fraction", [(3, 0.5), (8, 0.9)])
def test_unequal_batches_reuse_slots_and_pages(models, name, dtype, batch_size, fraction):
    """Batches one after another in a cache sized for one: slots, pages and state rows are used again, and a
    request's logits do not depend on its neighbours (compared with the plain run of each alone)."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name] + LENGTHS[name][::-1], 5)
    check(models, name, dtype, replay.batched(reqs, batch_size, fraction), reqs, "batched")


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_steps(models, name, dtype):
    """Steps that carry a fresh prompt, a later portion of another and single tokens side by side."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 6)
    check(models, name, dtype, replay.mixed(reqs), reqs, "mixed")


def test_a_freed_state_row_starts_from_zero(models):
    """A sequence that takes over a slot must not see the convolution rows or the recurrent state left there."""
    eng, cfg, w, _ = models[("M4", "float32")]
    reqs = requests_for(cfg, [40, 6], 8)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"], "want": [39]}], "end": ["r0"]},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"], "want": list(range(6))}], "end": ["r1"]}]
    got = replay.run_in_process(eng, steps, max_tokens=64)
    want = plain_logits(cfg, w, reqs)
    replay.compare(got, {k: v for k, v in want.items() if k in got}, "float32", "slot reuse")


@pytest.mark.parametrize("name", ["M1", "M3"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_greedy_generation_through_the_entry_point(models, name, use_graph):
    """Engine.generate (scheduler, batches, captured decode steps) against the plain greedy loop."""
    eng, cfg, w, _ = models[(name, "float32")]
    prompts = list(requests_for(cfg, [5, 1, 19, 66], 9).values())
    outs = eng.generate(prompts, max_tokens=[12, 20, 7, 9], temperature=0.0, use_graph=use_graph, stop_token_ids=[])
    for p, o, n in zip(prompts, outs, [12, 20, 7, 9]):
        assert o == plain.generate(p, n, w, cfg), (len(p), o)


def test_trace_replay_program(models, tmp_path):
    eng, cfg, w, folder = models[("M3", "float32")]
    reqs = requests_for(cfg, [40, 3, 77], 10)
    steps = replay.batched(reqs, 3, 0.6)
    got = replay.run_binary(folder, "float32", steps, str(tmp_path / "out"), cfg["vocab"])
    replay.compare(got, plain_logits(cfg, w, reqs), "float32", "bin/trace_run")


def test_command_line_generates(models):
    import json, os, subprocess, sys
    eng, cfg, w, folder = models[("M2", "float32")]
    out = subprocess.run([sys.executable, "-m", "pico_engine", folder, "--prompt", "5,17,3", "--max-tokens", "6", "--temperature", "0",
                          "--dtype", "float32"], capture_output=True, text=True, cwd=replay.ROOT, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    assert json.loads(line)["output"] == plain.generate([5, 17, 3], 6, w, cfg)


# ------------------------------------------------------------------ attention with mixed heads, alone

def paged(k, v, dtype, order_seed=0):
    """Keys and values of one sequence [n, G, D] / [n, G, Dv] in cache pools whose pages lie in a scrambled order."""
    n, G, D = k.shape
    Dv = v.shape[2]
    pages = (n + 63) // 64
    phys = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(order_seed))[:pages]
    kp = torch.full((pages + 3, G, 64, D), 7.0)
    vp = torch.full((pages + 3, G, 64, Dv), -7.0)
    for p in range(n):
        kp[phys[p // 64], :, p % 64] = k[p]
        vp[phys[p // 64], :, p % 64] = v[p]
    return kp.to(dtype).cuda(), vp.to(dtype).cuda(), phys.to(torch.int32).view(1, -1).cuda()


def run_headmix(q, k, v, scale, sink, talk, window, dtype, decode_last=0):
    """The kernel on one sequence: all tokens as one prompt step, or the last ``decode_last`` tokens each as a step of its own."""
    from pico_engine.ops import kernels
    n, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    kp, vp, table = paged(k, v, dtype)
    dev = lambda t: None if t is None else t.float().cuda().contiguous()
    outs = []
    spans = [(0, n)] if not decode_last else [(p, p + 1) for p in range(n - decode_last, n)]
    for a, b in spans:
        ctx = SimpleNamespace(one_token_each=(b - a == 1), scratch={}, lens=[b - a], starts=[a], max_context=b)
        pos = torch.arange(a, b, dtype=torch.int32).cuda()
        row = torch.zeros(b - a, dtype=torch.int32).cuda()
        qq = q[a:b].reshape(b - a, H * D).to(dtype).cuda().contiguous()
        outs.append(kernels.attention_headmix(qq, H * D, H, G, D, Dv, kp, vp, table, table.shape[1], pos, row, window, scale,
                                              dev(sink), dev(talk), ctx).float().cpu().view(b - a, H, Dv))
    return torch.cat(outs)


def rounded(t, dtype):
    return t.to(dtype).double()


@pytest.mark.parametrize("dtype,path", [("float32", "1"), ("bfloat16", "1"), ("bfloat16", "two-pass"), ("bfloat16", "0")])
@pytest.mark.parametrize("H,G,D,Dv", [(4, 2, 32, 16), (3, 3, 16, 40), (8, 1, 24, 24), (1, 1, 64, 8), (12, 4, 64, 64)])
def test_headmix_kernel_random(monkeypatch, dtype, path, H, G, D, Dv):
    """All three bfloat16 kernels (one pass on the tensor cores, two passes on the tensor cores, float32 FMAs) and the
    float32 one, in a prompt and in single-token steps."""
    from pico_engine.ops import kernels
    monkeypatch.setattr(kernels, "HEADMIX_TENSOR_CORES", path)
    g = torch.Generator().manual_seed(H * 100 + D)
    n = 150
    dt = DTYPES[dtype]
    q, k, v = (rounded(torch.randn(n, h, d, generator=g), dt) for h, d in ((H, D), (G, D), (G, Dv)))
    sink, talk = torch.randn(H, generator=g).double(), (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)).double()
    want = plain.mixed_attention(q, k, v, 0.3, sink, talk)
    tol = (2e-5 if dtype == "float32" else 1.5e-2) * max(1.0, float(want.abs().max()))
    assert (run_headmix(q, k, v, 0.3, sink, talk, None, dt) - want).abs().max() < tol
    assert (run_headmix(q, k, v, 0.3, sink, talk, None, dt, decode_last=20) - want[-20:]).abs().max() < tol
    # without a sink and without mixing it is plain grouped attention
    want = plain.mixed_attention(q, k, v, 0.3, None, None)
    assert (run_headmix(q, k, v, 0.3, None, None, None, dt) - want).abs().max() < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,far", [(700, 0), (700, 1), (700, 63), (700, 64), (700, 447), (129, 127), (129, 128), (65, 31), (65, 32), (33, 32)])
def test_headmix_kernel_finds_one_key_among_hundreds(n, far, dtype):
    """One key is made to match the last queries and carries a value nobody else has: the output must be that
    value (times what the sink leaves), in a prompt and in single-token steps, wherever the key lies: the first
    positions, the borders of a page (63/64, 127/128) and of a block of 32 keys."""
    H, G, D, Dv = 4, 2, 16, 8
    g = torch.Generator().manual_seed(n + far)
    q, k, v = 0.1 * torch.randn(n, H, D, generator=g), 0.1 * torch.randn(n, G, D, generator=g), torch.randn(n, G, Dv, generator=g)
    mark = torch.zeros(D); mark[3] = 6.0
    k[far] = mark
    q[-5:] = mark
    v[far] = 50.0
    dt = DTYPES[dtype]
    q, k, v = rounded(q, dt), rounded(k, dt), rounded(v, dt)
    sink = torch.full((H,), -2.0).double()
    talk = torch.tensor([[0, 1, 0, 0], [1, 0, 0, 0], [0, 0, 0.5, 0.5], [0, 0, 1, -1]], dtype=torch.float64)
    want = plain.mixed_attention(q, k, v, 1.0, sink, talk)
    assert want[-1, 0, 0] > 49 and abs(float(want[-1, 3, 0])) < 1          # heads 0-2 see the key alone, head 3's weights cancel
    for decode_last in (0, 5):
        got = run_headmix(q, k, v, 1.0, sink, talk, None, dt, decode_last)
        assert (got - want[-got.shape[0]:]).abs().max() < (1e-3 if dtype == "float32" else 0.3), (n, far, decode_last)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 31, 32, 33, 64, 100])
def test_headmix_kernel_window_edges(window, dtype):
    """A marked key ``window - 1`` places back is the oldest one seen, one place further back it is not."""
    H, G, D, Dv, n = 2, 1, 16, 8, 230
    g = torch.Generator().manual_seed(window)
    q, k, v = 0.1 * torch.randn(n, H, D, generator=g), 0.1 * torch.randn(n, G, D, generator=g), torch.randn(n, G, Dv, generator=g)
    mark = torch.zeros(D); mark[0] = 6.0
    at = 120
    k[at] = mark; v[at] = 40.0
    q[at:] = mark
    dt = DTYPES[dtype]
    q, k, v = rounded(q, dt), rounded(k, dt), rounded(v, dt)
    want = plain.mixed_attention(q, k, v, 1.0, None, None, window)
    assert want[at + window - 1, 0, 0] > 30 and abs(float(want[at + window, 0, 0])) < 5
    for decode_last in (0, 110):
        got = run_headmix(q, k, v, 1.0, None, None, window, dt, decode_last)
        assert (got - want[-got.shape[0]:]).abs().max() < (1e-3 if dtype == "float32" else 0.3), (window, decode_last)


def test_headmix_kernel_sink_alone_scales_the_output():
    """With one key the weight is e^s / (e^s + e^sink): a large sink takes nearly everything, a very small one nothing."""
    q = torch.ones(1, 2, 16).double(); k = torch.ones(1, 1, 16).double(); v = torch.ones(1, 1, 8).double()
    for sink in (-30.0, 0.0, 1.6, 30.0):
        got = run_headmix(q, k, v, 0.1, torch.tensor([sink, 1.6]), None, None, torch.float32)
        assert abs(float(got[0, 0, 0]) - 1 / (1 + math.exp(sink - 1.6))) < 1e-6 and abs(float(got[0, 1, 0]) - 0.5) < 1e-6


# ------------------------------------------------------------------ the recurrence, alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunked", [False, True])
def test_mingru_kernel_packed_sequences_and_carried_state(dtype, chunked):
    """Packed sequences whose borders fall inside and on the borders of a chunk, in two steps: the second step
    continues every sequence from the state the first one left in its slot."""
    from pico_engine.ops import kernels
    dt, W = DTYPES[dtype], 70
    g = torch.Generator().manual_seed(5)
    lens1, lens2, slots = [1, 33, 64, 2, 31], [40, 1, 3, 32, 1], [4, 0, 2, 5, 1]
    proj = {s: rounded(2 * torch.randn(a + b, 3 * W, generator=g), dt) for s, a, b in zip(slots, lens1, lens2)}
    state = torch.full((7, W + 5), 3.0).cuda()           # the part's numbers lie at offset 5 of each slot's row
    state[:, 5:] = 0
    outs = {s: [] for s in slots}
    for step, lens in enumerate((lens1, lens2)):
        rows = [proj[s][:a] if step == 0 else proj[s][a:] for s, a in zip(slots, lens1)]
        first = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        tok_row = np.repeat(np.arange(len(lens)), lens).astype(np.int32)
        y = kernels.mingru(torch.cat(rows).to(dt).cuda().contiguous(), state, 5, torch.from_numpy(tok_row).cuda(),
                           torch.from_numpy(first).cuda(), torch.tensor(lens, dtype=torch.int32).cuda(),
                           torch.tensor(slots, dtype=torch.int32).cuda(), chunked=chunked).float().cpu()
        for b, s in enumerate(slots):
            outs[s].append(y[first[b]:first[b + 1]])
    tol = 1e-5 if dtype == "float32" else 3e-2
    for s in slots:
        want, S = plain.mingru_recurrence(proj[s][:, :W], proj[s][:, W:2 * W], proj[s][:, 2 * W:])
        assert (torch.cat(outs[s]) - want).abs().max() < tol * max(1.0, float(want.abs().max()))
        assert (state[s, 5:].cpu() - S).abs().max() < 1e-5
    assert float(state[:, :5].min()) == 3.0 and float(state[3].abs().max()) == 3.0        # nothing else was written


# ------------------------------------------------------------------ norm and input convolution, alone

@pytest.mark.parametrize("taps", [1, 2, 3, 5])
@pytest.mark.parametrize("fused", [True, False])
def test_layernorm_and_convolution_across_steps(taps, fused):
    """Two sublayers read the same rows; sequences come in steps of 1, 2 and more tokens, so rows before a step's
    first token come from the state, also when a step is shorter than the convolution reaches back."""
    from pico_engine.ops import kernels
    H, eps = 50, 1e-5
    g = torch.Generator().manual_seed(taps)
    cuts = {2: [1, 1, 2, 1, 7, 3], 0: [9, 1, 1, 1, 2], 3: [2, 30, 1]}           # slot -> tokens brought in consecutive steps
    x = {s: 3 * torch.randn(sum(c), H, generator=g) + 1.0 for s, c in cuts.items()}
    par = [(1 + 0.1 * torch.randn(H, generator=g), torch.randn(H, generator=g), torch.randn(H, taps, generator=g)) for _ in range(2)]
    hist = (taps - 1) * H
    state = torch.zeros(4, 3 + 2 * hist).cuda()
    offs = [3, 3 + hist]
    got = {s: [[], []] for s in cuts}
    dev = [tuple(t.cuda() for t in p) for p in par]
    for step in range(max(len(c) for c in cuts.values())):
        live = [s for s, c in cuts.items() if step < len(c)]
        lens = [cuts[s][step] for s in live]
        at = [sum(cuts[s][:step]) for s in live]
        rows = torch.cat([x[s][a:a + n] for s, a, n in zip(live, at, lens)]).cuda().contiguous()
        first = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).cuda()
        tok_row = torch.from_numpy(np.repeat(np.arange(len(lens)), lens).astype(np.int32)).cuda()
        ln, sl = torch.tensor(lens, dtype=torch.int32).cuda(), torch.tensor(live, dtype=torch.int32).cuda()
        if fused:
            outs = kernels.dual_layernorm_conv(rows, [(w, b, c, o) for (w, b, c), o in zip(dev, offs)], eps, state, tok_row, first,
                                               ln, sl, torch.float32, all(n == 1 for n in lens))
        else:
            outs = [kernels.causal_conv_add(kernels.layernorm(rows, w, b, eps, torch.float32), c, state, o, tok_row, first, ln, sl,
                                            torch.float32) for (w, b, c), o in zip(dev, offs)]
        for b, s in enumerate(live):
            for half in range(2):
                got[s][half].append(outs[half][int(first[b]):int(first[b + 1])].cpu())
    for s in cuts:
        for half, (w, b, c) in enumerate(par):
            want = plain.input_conv(plain.layer_norm(x[s].double(), w.double(), b.double(), eps), c.double())
            assert (torch.cat(got[s][half]) - want).abs().max() < 2e-5 * max(1.0, float(want.abs().max())), (s, half)
    assert float(state[:, :3].abs().max()) == 0 and float(state[1].abs().max()) == 0


def test_pointwise_kernels():
    from pico_engine.ops import kernels
    v = torch.linspace(-6, 6, 1001)
    for kind, fn in (("relu2", lambda t: torch.relu(t) ** 2), ("gelu_tanh", plain.gelu_tanh), ("silu", lambda t: t * torch.sigmoid(t))):
        assert (kernels.activation(v.cuda(), kind).cpu() - fn(v.double())).abs().max() < 1e-5
    lg = torch.linspace(-80, 80, 4000).cuda().view(4, 1000).contiguous()
    want = 11.0 * torch.tanh(lg.double().cpu() / 11.0)
    assert (kernels.softcap(lg, 11.0).cpu() - want).abs().max() < 1e-5
    pos = torch.tensor([0, 1, 77, 4095, 100000], dtype=torch.int32).cuda()
    for width in (10, 7):
        freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange((width + 1) // 2, dtype=torch.float64) / width)
        x = torch.ones(5, width).cuda()
        want = torch.stack([1 + plain.sinusoid(1, width, torch.float64, first=int(p))[0] for p in pos.cpu()])
        assert (kernels.add_sinusoid(x, pos, freq.float().cuda()).cpu() - want).abs().max() < 5e-3      # the angle is a float32 product
        assert (x[:3].cpu() - want[:3]).abs().max() < 1e-5
