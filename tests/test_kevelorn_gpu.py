"""Kevelorn on the GPU against the plain implementation: each mechanism's kernel alone on inputs that show a fault,
and the whole model through the library's step function, cache, scheduler and entry points, in both dtypes, for
every way of cutting requests into steps."""
from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_kevelorn as plain
import replay
from conftest import write_model
from kevelorn_models import CONFIGS, RANKS, make_weights, plain_logits, requests_for

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
CASES = [(n, d) for n in sorted(CONFIGS) for d in ("float32", "bfloat16")]
LENGTHS = {"K1": [1, 2, 3, 37, 70, 131, 64, 5], "K2": [65, 1, 150, 9, 33, 2], "K3": [3, 129, 31, 64, 1, 200], "K4": [4, 1, 90, 17, 66]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{(config, dtype): (engine, cfg, weights, folder)}."""
    from pico_engine.engine.engine import Engine
    root = tmp_path_factory.mktemp("kevelorn")
    out = {}
    for k, (name, cfg) in enumerate(sorted(CONFIGS.items())):
        weights = make_weights(cfg, 40 + k, RANKS[name])
        folder = write_model(root / name, cfg, weights)
        for dtype in DTYPES:
            out[(name, dtype)] = (Engine(folder, dtype=dtype), cfg, weights, folder)
    return out


def compare(got, cfg, w, reqs, dtype, what, only_got=False):
    """Against the plain logits; in bfloat16 without the places where the plain router's choice was a close call."""
    close = set()
    want = plain_logits(cfg, w, reqs, close)
    if only_got:
        want = {k: v for k, v in want.items() if k in got}
    if dtype == "bfloat16":
        assert len(close) < 0.5 * len(want)
        got, want = ({k: v for k, v in d.items() if k not in close} for d in (got, want))
    replay.compare(got, want, dtype, what)


def check(models, name, dtype, steps, reqs, what):
    eng, cfg, w, _ = models[(name, dtype)]
    compare(replay.run_in_process(eng, steps), cfg, w, reqs, dtype, what)


# ------------------------------------------------------------------ the whole model, every way of cutting

@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_and_first_tokens(models, name, dtype):
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 1)
    check(models, name, dtype, replay.whole(reqs), reqs, "whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(models, name, dtype):
    """Every request again with its last tokens one at a time (the shortest ones entirely), 100 for the long ones:
    the windows pass over decoded tokens, and the states are carried from token to token."""
    reqs = requests_for(CONFIGS[name], LENGTHS[name], 2)
    check(models, name, dtype, replay.tail(reqs, 100), reqs, "tail")


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompts_in_portions(models, name, dtype):
    """Portions of unequal sizes, then portions of two, three and five tokens and single tokens in turn: every
    portion starts inside its sequence from the state and the cache pages the portion before it left."""
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


@pytest.mark.parametrize("name,dtype", [("K1", "float32"), ("K1", "bfloat16"), ("K3", "bfloat16"), ("K4", "float32")])
def test_batches_of_more_rows_than_the_decode_products_fuse(models, name, dtype):
    """Twenty short requests start together and are decoded together: steps of 17 and more rows take the products and the
    residual sums that prompts take, and the recurrence walks twenty sequences side by side."""
    reqs = requests_for(CONFIGS[name], [3 + (7 * i) % 23 for i in range(20)], 13)
    check(models, name, dtype, replay.batched(reqs, 20, 0.5), reqs, "twenty rows")


@pytest.mark.parametrize("name", ["K1", "K2"])
def test_long_decoding(models, name):
    """300 tokens one by one from a one-token prompt: windows, pages given back, and states over many steps."""
    reqs = requests_for(CONFIGS[name], [301], 12)
    check(models, name, "float32", replay.tail(reqs, 300), reqs, "long decoding")


def test_a_freed_state_row_starts_from_zero(models):
    """A sequence that takes over a slot must not see the matrix states left there."""
    eng, cfg, w, _ = models[("K1", "float32")]
    reqs = requests_for(cfg, [40, 6], 8)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"], "want": [39]}], "end": ["r0"]},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"], "want": list(range(6))}], "end": ["r1"]}]
    got = replay.run_in_process(eng, steps, max_tokens=64)
    compare(got, cfg, w, reqs, "float32", "slot reuse", only_got=True)


@pytest.mark.parametrize("name", ["K1", "K3"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_greedy_generation_through_the_entry_point(models, name, use_graph):
    """Engine.generate (scheduler, batches, captured decode steps) against the plain greedy loop."""
    eng, cfg, w, _ = models[(name, "float32")]
    w64 = {n: t.double() for n, t in w.items()}
    prompts = list(requests_for(cfg, [5, 1, 19, 66], 9).values())
    outs = eng.generate(prompts, max_tokens=[12, 20, 7, 9], temperature=0.0, use_graph=use_graph, stop_token_ids=[])
    for p, o, n in zip(prompts, outs, [12, 20, 7, 9]):
        assert p + o == plain.generate(p, w64, cfg, n), (len(p), o)


def test_bfloat16_generation_with_graphs_matches_eager(models):
    eng, cfg, w, _ = models[("K4", "bfloat16")]
    prompts = list(requests_for(cfg, [7, 30, 2], 11).values())
    a = eng.generate(prompts, max_tokens=10, temperature=0.0, use_graph=False, stop_token_ids=[])
    b = eng.generate(prompts, max_tokens=10, temperature=0.0, use_graph=True, stop_token_ids=[])
    assert a == b


def test_trace_replay_program(models, tmp_path):
    eng, cfg, w, folder = models[("K2", "float32")]
    reqs = requests_for(cfg, [40, 3, 77], 10)
    steps = replay.batched(reqs, 3, 0.6)
    got = replay.run_binary(folder, "float32", steps, str(tmp_path / "out"), cfg["vocab"])
    compare(got, cfg, w, reqs, "float32", "bin/trace_run")


def test_command_line_generates(models):
    import json, subprocess, sys
    eng, cfg, w, folder = models[("K3", "float32")]
    out = subprocess.run([sys.executable, "-m", "pico_engine", folder, "--prompt", "5,17,3", "--max-tokens", "6", "--temperature", "0",
                          "--dtype", "float32"], capture_output=True, text=True, cwd=replay.ROOT, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    assert [5, 17, 3] + json.loads(line)["output"] == plain.generate([5, 17, 3], {n: t.double() for n, t in w.items()}, cfg, 6)


# ------------------------------------------------------------------ the recurrence, alone

def run_recurrence(q, k, v, dtype, lens, head_decay=None, logits=None, tau=1.0, q_scale=1.0, act="none", cuts=(1.0,), chunked=None):
    """The kernel on packed sequences of ``lens`` tokens, brought in steps that cut every sequence at the fractions
    ``cuts``; q, k [T, H, D], v [T, H, Dv] hold the sequences one after another.  Returns o [T, H, Dv] and the states."""
    from pico_engine.ops import kernels
    T, H, D = q.shape
    Dv = v.shape[2]
    B = len(lens)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(dtype).cuda().contiguous()
    z = None if logits is None else logits.reshape(T, H * D).float().cuda().contiguous()
    hd = None if head_decay is None else torch.tensor(head_decay, dtype=torch.float32).cuda()
    state = torch.full((B + 2, 5 + H * D * Dv), 3.0).cuda()               # the part's state begins at offset 5 of a slot's row
    slots = torch.tensor([b + 1 for b in range(B)], dtype=torch.int32).cuda()
    state[1:B + 1, 5:] = 0
    first = np.concatenate([[0], np.cumsum(lens)])
    out = torch.zeros(T, H * Dv)
    done = [0] * B
    for c in cuts:
        upto = [n if c == cuts[-1] else max(d, int(n * c)) for n, d in zip(lens, done)]
        rows = [b for b in range(B) if upto[b] > done[b]]
        idx = torch.cat([torch.arange(first[b] + done[b], first[b] + upto[b]) for b in rows])
        step_lens = [upto[b] - done[b] for b in rows]
        rf = torch.tensor(np.concatenate([[0], np.cumsum(step_lens)]), dtype=torch.int32).cuda()
        rl = torch.tensor(step_lens, dtype=torch.int32).cuda()
        use_chunks = (len(idx) > 2 * len(rows)) if chunked is None else chunked
        o = kernels.linear_attention(proj[idx.cuda()].contiguous(), 0, H * D, 2 * H * D, H, D, Dv, state, 5, rf, rl,
                                     slots[torch.tensor(rows).cuda()].contiguous(), use_chunks, head_decay=hd,
                                     decay_logits=None if z is None else z[idx.cuda()].contiguous(), inv_tau=1.0 / tau,
                                     q_scale=q_scale, qk_activation=act, v_activation=act)
        out[idx] = o.cpu()
        done = upto
    assert float(state[0].min()) == 3.0 and float(state[B + 1].min()) == 3.0 and float(state[:, :5].min()) == 3.0
    return out.view(T, H, Dv), state[1:B + 1, 5:].cpu().view(B, H, D, Dv)


def plain_recurrence(q, k, v, lens, decay):
    outs, states, at = [], [], 0
    for n in lens:
        o, S = plain.linear_recurrence(q[at:at + n].double(), k[at:at + n].double(), v[at:at + n].double(), decay[at:at + n].double())
        outs.append(o); states.append(S); at += n
    return torch.cat(outs), torch.stack(states)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,Dv", [(2, 16, 8), (3, 24, 40), (1, 64, 64), (2, 136, 12), (4, 128, 33), (1, 200, 96), (2, 128, 128), (1, 96, 72),
                                    (3, 40, 100)])
def test_recurrence_kernel_fixed_decay(dtype, H, D, Dv):
    """Sequences whose lengths fall on, before and after chunk borders, as one prompt step (chunked and token after token),
    in portions, and with the last tokens one by one; the states are compared too."""
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(H * 1000 + D)
    lens = [1, 64, 65, 130, 2, 63, 200]
    T = sum(lens)
    q, k, v = ((torch.randn(T, H, d, generator=g) * d ** -0.25).to(dt).float() for d in (D, D, Dv))
    decay = [0.3, 1.0, 0.97, 0.999][:H] if H <= 4 else None
    dec = torch.tensor(decay).view(1, H, 1).expand(T, H, D)
    want_o, want_s = plain_recurrence(q, k, v, lens, dec)
    tol = (1e-5 if dtype == "float32" else 1e-5) * max(1.0, float(want_o.abs().max()))       # the inputs are the same rounded values
    for cuts, chunked in (((1.0,), True), ((1.0,), False), ((0.4, 0.75, 1.0), None), ((0.97, 0.98, 0.99, 1.0), None)):
        o, s = run_recurrence(q, k, v, dt, lens, head_decay=decay, cuts=cuts, chunked=chunked)
        assert (o.double() - want_o).abs().max() < tol, (cuts, chunked)
        assert (s.double() - want_s).abs().max() < tol * 10, (cuts, chunked)


@pytest.mark.parametrize("H,D,Dv,tau", [(2, 16, 8, 1.0), (3, 48, 32, 16.0), (1, 136, 24, 4.0), (2, 80, 64, 8.0), (1, 128, 160, 2.0)])
def test_recurrence_kernel_decay_per_channel(H, D, Dv, tau):
    """A learned decay per key channel and token, query scale and silu on the projections."""
    g = torch.Generator().manual_seed(D)
    lens = [70, 3, 129]
    T = sum(lens)
    q, k, v = (torch.randn(T, H, d, generator=g) for d in (D, D, Dv))
    z = 2.0 * torch.randn(T, H, D, generator=g) + 1.0
    alpha = plain.sigmoid(z.double()) ** (1.0 / tau)
    want_o, want_s = plain_recurrence(plain.silu(q.double()) * 0.25, plain.silu(k.double()), plain.silu(v.double()), lens, alpha)
    for cuts, chunked in (((1.0,), True), ((1.0,), False), ((0.5, 1.0), None)):
        o, s = run_recurrence(q, k, v, torch.float32, lens, logits=z, tau=tau, q_scale=0.25, act="silu", cuts=cuts, chunked=chunked)
        assert (o.double() - want_o).abs().max() < 2e-5 * max(1.0, float(want_o.abs().max())), (cuts, chunked)
        assert (s.double() - want_s).abs().max() < 2e-4 * max(1.0, float(want_s.abs().max()))


@pytest.mark.parametrize("far", [0, 1, 63, 64, 65, 447])
def test_recurrence_keeps_a_key_from_far_back(far):
    """With decay 1 one key that matches the last query and carries a value nobody else has must come through whole
    from any distance: the first positions, chunk borders, hundreds of tokens back."""
    H, D, Dv, n = 1, 16, 8, 700
    g = torch.Generator().manual_seed(far)
    q, k, v = 0.01 * torch.randn(n, H, D, generator=g), 0.001 * torch.randn(n, H, D, generator=g), torch.randn(n, H, Dv, generator=g)
    k[far, 0] = 0; k[far, 0, 3] = 10.0
    q[-1, 0] = 0; q[-1, 0, 3] = 10.0
    v[far, 0] = 50.0                                           # the other 699 keys together add about 0.3 to the 5000
    for cuts in ((1.0,), (0.5, 0.999, 1.0)):
        o, _ = run_recurrence(q, k, v, torch.float32, [n], head_decay=[1.0], cuts=cuts)
        assert (o[-1, 0] - 5000.0).abs().max() < 2.0, (far, cuts, o[-1, 0])


# ------------------------------------------------------------------ rotation, unit norm and the cache write; the window

@pytest.mark.parametrize("pad", [5, 6])          # rows of odd and of even length (the latter let a lane take whole pairs)
@pytest.mark.parametrize("D", [24, 80, 200])
def test_rotation_norm_and_store(D, pad):
    from pico_engine.ops import kernels
    H, G, Dv, n = 3, 1, 40, 70
    g = torch.Generator().manual_seed(3)
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        for dims, norm in ((D, True), (8, True), (0, True), (16, False)):
            row = torch.randn(n, H * D + G * D + G * Dv + pad, generator=g).to(dtype)
            pos = torch.arange(100, 100 + n, dtype=torch.int32)
            freq = (50.0 ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / max(dims, 1)) / 3.0).float()
            kp, vp = torch.zeros(4, G, 64, D, dtype=dtype).cuda(), torch.zeros(4, G, 64, Dv, dtype=dtype).cuda()
            table = torch.tensor([[-1, 2, 0]], dtype=torch.int32).cuda()
            dev = row.cuda().contiguous()
            kernels.rotary_norm_store(dev, H, G, D, Dv, freq.cuda() if dims else None, dims, norm, 1e-5, pos.cuda(),
                                      torch.zeros(n, dtype=torch.int32).cuda(), kp, vp, table, 3)
            x = row.double()
            heads = x[:, :(H + G) * D].view(n, H + G, D)
            want = heads if not dims else plain.rotate_pairs(heads, 100, dims, 50.0, 3.0)
            # the oracle's frequencies are float64; the kernel's were rounded to float32: angles near 170 differ by 1e-5
            want = plain.rms_unit(want, 1e-5) if norm else want
            got = dev.cpu().double()
            assert (got[:, :(H + G) * D].view(n, H + G, D) - want).abs().max() < max(tol, 3e-5) * 4
            assert torch.equal(got[:, (H + G) * D:], x[:, (H + G) * D:])                      # values and the rest stay
            for t in (0, 27, 28, 69):                                                         # positions 100, 127 | 128, 169
                p = 100 + t
                page = int(table[0, p // 64])
                assert torch.equal(kp[page, :, p % 64].cpu().double().view(-1), got[t, H * D:(H + G) * D])
                assert torch.equal(vp[page, :, p % 64].cpu().double().view(-1), got[t, (H + G) * D:(H + G) * D + G * Dv])


@pytest.mark.parametrize("name,dtype", [("K1", "float32"), ("K1", "bfloat16"), ("K2", "bfloat16"), ("K2", "float32"), ("K4", "float32"), ("K4", "bfloat16")])
def test_window_edge_in_prompt_and_decoding(models, name, dtype):
    """The softmax mixer of a model alone: one key is made to dominate for the queries that follow it; it must be seen by
    the query window - 1 places after it and not by the next one, in a prompt step and token by token, with the key on
    either side of a page border."""
    from pico_engine.config.specs import GatedAttentionSpec
    eng, cfg, _, _ = models[(name, dtype)]
    layer = next(l for l in cfg["layers"] if l["type"] == "parallel")["mixer"]["left"]
    window, H, G, D, Dv = layer["mask"]["size"], layer["heads"], layer["kv_heads"], layer["dim"], layer["vdim"]
    from pico_engine.parts.attention_gated import GatedAttention
    from pico_engine.config.specs import NoPositionSpec
    part = GatedAttention(GatedAttentionSpec(hidden=8, n_heads=H, n_kv_heads=G, head_dim=D, v_head_dim=Dv, window=window, scale=1.0,
                                             position=NoPositionSpec(), prefix="", gate=None), DTYPES[dtype], "cuda")
    from pico_engine.ops import kernels
    for key_at in (5, 63, 64, 100):
        n = key_at + window + 3
        g = torch.Generator().manual_seed(key_at)
        q, k, v = 0.01 * torch.randn(n, H, D, generator=g), 0.01 * torch.randn(n, G, D, generator=g), torch.randn(n, G, Dv, generator=g)
        k[key_at] = 0; k[key_at, :, 1] = 6.0
        q[key_at + 1:] = 0; q[key_at + 1:, :, 1] = 6.0
        v[key_at] = 100.0
        dt = DTYPES[dtype]
        pages = (n + 63) // 64
        kp, vp = torch.zeros(pages + 1, G, 64, D, dtype=dt).cuda(), torch.zeros(pages + 1, G, 64, Dv, dtype=dt).cuda()
        for p in range(n):
            kp[1 + p // 64, :, p % 64] = k[p].to(dt).cuda(); vp[1 + p // 64, :, p % 64] = v[p].to(dt).cuda()
        table = torch.arange(1, pages + 1, dtype=torch.int32).view(1, -1).cuda()
        for spans in ([(0, n)], [(p, p + 1) for p in range(key_at + 1, n)]):
            for a, b in spans:
                ctx = SimpleNamespace(one_token_each=(b - a == 1), scratch={}, lens=[b - a], starts=[a], max_context=b, dtype=dt)
                pos, row = torch.arange(a, b, dtype=torch.int32).cuda(), torch.zeros(b - a, dtype=torch.int32).cuda()
                qq = q[a:b].reshape(b - a, H * D).to(dt).cuda().contiguous()
                if part.plain_kernels:
                    o = kernels.attention(qq, H * D, H, G, D, kp, vp, table, pages, pos, row, window, 1.0, ctx)
                else:
                    o = kernels.attention_headmix(qq, H * D, H, G, D, Dv, kp, vp, table, pages, pos, row, window, 1.0, None, None, ctx)
                o = o.float().cpu().view(b - a, H, Dv)
                for p in range(max(a, key_at + 1), b):
                    seen = p - key_at < window
                    assert (o[p - a].min() > 90.0) == seen and (o[p - a].max() < 10.0) == (not seen), (key_at, p, seen, o[p - a].min(), o[p - a].max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [32, 48])
def test_a_window_of_one_sees_only_the_token_itself(dtype, D):
    from pico_engine.ops import kernels
    dt = DTYPES[dtype]
    H, G, n = 4, 2, 140
    g = torch.Generator().manual_seed(D)
    q, k, v = torch.randn(n, H, D, generator=g), torch.randn(n, G, D, generator=g), torch.randn(n, G, D, generator=g).to(dt).float()
    pages = (n + 63) // 64
    kp, vp = torch.zeros(pages + 1, G, 64, D, dtype=dt).cuda(), torch.zeros(pages + 1, G, 64, D, dtype=dt).cuda()
    for p in range(n):
        kp[1 + p // 64, :, p % 64] = k[p].to(dt).cuda(); vp[1 + p // 64, :, p % 64] = v[p].to(dt).cuda()
    table = torch.arange(1, pages + 1, dtype=torch.int32).view(1, -1).cuda()
    for spans in ([(0, n)], [(p, p + 1) for p in (0, 1, 63, 64, 139)]):
        for a, b in spans:
            ctx = SimpleNamespace(one_token_each=(b - a == 1), scratch={}, lens=[b - a], starts=[a], max_context=b, dtype=dt)
            pos, row = torch.arange(a, b, dtype=torch.int32).cuda(), torch.zeros(b - a, dtype=torch.int32).cuda()
            o = kernels.attention(q[a:b].reshape(b - a, H * D).to(dt).cuda().contiguous(), H * D, H, G, D, kp, vp, table, pages, pos, row, 1, 0.3, ctx)
            want = v[a:b].repeat_interleave(H // G, dim=1)
            assert (o.float().cpu().view(b - a, H, D) - want).abs().max() < 1e-2


# ------------------------------------------------------------------ norms with gates, sums of branches, the stream

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,Dv,off", [(9, 3, 40, 7), (9, 3, 40, 8), (5, 6, 128, 0), (3, 1, 4100, 4), (4, 5, 6, 3)])
def test_gated_norm_kernel(dtype, T, H, Dv, off):
    """Norm over all heads, per head and no norm, times the gate: rows that are and are not aligned for vector accesses, runs that
    a warp, a block with registers, and a block with a loop take."""
    from pico_engine.ops import kernels
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(1)
    o = torch.randn(T, H * Dv, generator=g) * 3
    gate = torch.randn(T, off + H * Dv, generator=g).to(dt)
    tol = 2e-6 if dtype == "float32" else 1e-2
    for group, act, fn in ((H * Dv, "sigmoid", plain.sigmoid), (Dv, "silu", plain.silu), (0, "sigmoid", plain.sigmoid)):
        w = (1 + 0.2 * torch.randn(max(group, 1), generator=g)).to(dt)
        src = o if group else o.to(dt)
        got = kernels.gated_norm(src.cuda(), group, w.cuda() if group else None, 1e-5, gate.cuda(), off, act, dt).float().cpu()
        x = src.double()
        if group:
            x = plain.norm_plain(x.view(T, -1, group), w.double(), 1e-5).reshape(T, H * Dv)
        want = x * fn(gate[:, off:].double())
        assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))
        if group:                                           # and without a gate
            got = kernels.gated_norm(src.cuda(), group, w.cuda(), 1e-5, None, 0, "none", dt).float().cpu()
            assert (got - x).abs().max() < tol * max(1.0, float(x.abs().max()))


@pytest.mark.parametrize("T,W", [(11, 50), (5, 72), (3, 1100)])          # widths that are and are not multiples of 4, below and above 1024
def test_branch_sum_scaled_add_and_stream_vectors(T, W):
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, W, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        ys = [(torch.randn(T, W, generator=g) * s).to(dt) for s in (1.0, 30.0, 0.01)]
        ws = [(1 + 0.3 * torch.randn(W, generator=g)).to(dt) for _ in ys]
        for n in (1, 2, 3):
            got = kernels.normed_sum_add(x.clone().cuda(), [y.cuda() for y in ys[:n]], [w.cuda() for w in ws[:n]], 1e-5, 0.15).cpu()
            want = x.double() + 0.15 * sum(plain.norm_plain(y.double(), w.double(), 1e-5) for y, w in zip(ys[:n], ws[:n]))
            assert (got - want).abs().max() < 3e-6
        got = kernels.scaled_add(x.clone().cuda(), ys[1].cuda(), 0.3).cpu()
        assert (got - (x.double() + 0.3 * ys[1].double())).abs().max() < 1e-5
        vec = torch.randn(W, generator=g).to(dt)
        rows = torch.randn(T, W, generator=g)
        assert (kernels.add_rows(x.clone().cuda(), rows.cuda(), vec.cuda()).cpu() - (x + rows + vec.float())).abs().max() < 1e-6
        assert (kernels.add_rows(x.clone().cuda(), None, vec.cuda()).cpu() - (x + vec.float())).abs().max() < 1e-6


# ------------------------------------------------------------------ routing and the gated activation

@pytest.mark.parametrize("E,top,extra", [(8, 4, True), (5, 1, False), (3, 3, True), (70, 6, False), (1, 1, True)])
def test_expert_choice(E, top, extra):
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(E)
    T = 37
    z = torch.randn(T, E + (1 if extra else 0), generator=g) * 3
    ids = torch.zeros(T, top, dtype=torch.int32).cuda()
    got = kernels.moe_route(z.cuda(), E, top, extra, ids).cpu()
    for t in range(T):
        order = sorted(range(E), key=lambda e: -float(z[t, e]))[:top]
        assert ids[t].tolist() == order
        p = torch.softmax(z[t, order].double(), 0)
        want = torch.zeros(E, dtype=torch.float64)
        want[order] = p
        assert (got[t, :E] - want).abs().max() < 1e-6
        assert sorted(torch.nonzero(got[t, :E]).view(-1).tolist()) == sorted(order)
        if extra:
            assert abs(float(got[t, E]) - 1 / (1 + math.exp(-float(z[t, E])))) < 1e-6


@pytest.mark.parametrize("E,top,extra,K", [(8, 4, True, 72), (3, 1, False, 50), (40, 5, True, 130)])
def test_expert_choice_from_the_stream(E, top, extra, K):
    """Norm, router product and choice in one kernel against the plain norm and router."""
    from pico_engine.ops import kernels
    g = torch.Generator().manual_seed(K)
    T = 21
    x = torch.randn(T, K, generator=g) * 3
    nw = 1 + 0.2 * torch.randn(K, generator=g)
    router = torch.randn(E + (1 if extra else 0), K, generator=g) * 3 * K ** -0.5
    ids = torch.zeros(T, top, dtype=torch.int32).cuda()
    got = kernels.moe_route_stream(x.cuda(), nw.cuda(), 1e-3, router.cuda(), E, top, extra, ids).cpu()
    z = plain.lin(router.double(), plain.norm_plain(x.double(), nw.double(), 1e-3))
    for t in range(T):
        order = sorted(range(E), key=lambda e: -float(z[t, e]))[:top]
        assert ids[t].tolist() == order
        want = torch.zeros(E, dtype=torch.float64)
        want[order] = torch.softmax(z[t, order], 0)
        assert (got[t, :E] - want).abs().max() < 1e-5
        if extra:
            assert abs(float(got[t, E]) - float(plain.sigmoid(z[t, E]))) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_activation_with_expert_weights(dtype):
    from pico_engine.ops import kernels
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(4)
    T, E, ff, shared = 6, 3, 10, 7
    I = E * ff + shared
    gu = torch.randn(T, 2 * I, generator=g).to(dt)
    wts = torch.rand(T, E + 1, generator=g)
    wts[:, 1] = 0
    gu[0, ff + 2] = float("inf")                                     # a hidden unit of an expert that is not used stays out
    tol = 2e-6 if dtype == "float32" else 1e-2
    got = kernels.gated_act(gu.cuda(), "silu", wts.cuda(), ff).float().cpu()
    col = torch.tensor([min(c // ff, E) for c in range(I)])
    want = plain.silu(gu[:, :I].double()) * gu[:, I:].double() * wts.double()[:, col]
    want[:, ff:2 * ff] = 0
    assert (got - want).abs().max() < tol * 5
    got = kernels.gated_act(gu[1:].contiguous().cuda(), "gelu_tanh").float().cpu()
    want = plain.gelu_tanh(gu[1:, :I].double()) * gu[1:, I:].double()
    assert (got - want).abs().max() < tol * 5


def test_routing_of_a_model_picks_what_the_plain_router_picks(models):
    """The mixture part alone against the plain mixture, token by token."""
    eng, cfg, w, _ = models[("K1", "float32")]
    part = eng.model.layers[0].feed_forward
    g = torch.Generator().manual_seed(5)
    h = torch.randn(19, cfg["width"], generator=g)
    ctx = SimpleNamespace(dtype=torch.float32)
    got = part.apply(h.cuda(), ctx).cpu()
    want = plain.mixture(h.double(), {n: t.double() for n, t in w.items()}, "l0.mlp.", cfg["layers"][0]["mlp"])
    assert (got - want).abs().max() < 2e-5 * max(1.0, float(want.abs().max()))
