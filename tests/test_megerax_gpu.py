"""The Megerax design in the engine against its plain implementation
(plain_megerax.py): every mechanism alone, then whole models of three small
configurations that differ in every size and option, under every way of
cutting the same requests into steps."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import go_tinygrad_b200 as lib
import plain_llama
import plain_megerax as plain
from go_tinygrad_b200.cache import Cache
from go_tinygrad_b200.config.registry import find_architecture
from go_tinygrad_b200.engine import Model, StepEntry, step
from go_tinygrad_b200.kernels import ops
from go_tinygrad_b200.parts import PartSpec, Runtime, build_part, walk
from conftest import ROOT, assert_close
from test_megerax_config import SCALING, attention, delta, latent, layer
from test_parts_gpu import context

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda" if torch.cuda.is_available() and torch.cuda.device_count() else "cpu")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}

# P: heads that share keys in groups of three, values narrower and wider than keys, four, two and no taps, a
# window of 70 and one of 5 on borrowed keys, capped and uncapped scores, part of a head rotating under
# wavelength scaling, a delta layer whose heads share queries and keys and one with ranks named by the
# configuration, a latent layer without a feed-forward, a multiplier on the logits.
CONFIG_P = {
    "architecture": "Megerax", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "layers": [
        layer("attention", attention(6, 2, 24, 16, 0.2, conv=4, window=70, rot={"dims": 16, "base": 100.0, "scaling": SCALING},
                                     softcap=5.0), 100),
        layer("channel_delta", delta(4, 2, 24, 40, conv=2), 36),
        layer("latent_attention", latent(3, 16, 8, 24, 40, 24, 0.2, {"dims": 8, "base": 1000.0})),
        layer("attention", attention(6, 2, 24, 16, 0.3, conv=2, window=5, rot={"dims": 16, "base": 100.0, "scaling": SCALING},
                                     kv_from=0), 64),
        layer("channel_delta", delta(2, 2, 40, 12, decay_rank=8, gate_rank=16)),
    ],
}
# Q: sizes the tensor-core kernels take: heads of 64 and 128 channels with values as wide; a latent layer
# with a window and a rotated part of which half turns; attention without convolution, window, cap or
# scaling and the whole head rotating; two layers that read a third one's keys; one head of keys for four.
CONFIG_Q = {
    "architecture": "Megerax", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 1.5,
    "layers": [
        layer("latent_attention", latent(4, 64, 32, 64, 64, 48, 0.1, {"dims": 16, "base": 10000.0}, window=100), 256),
        layer("attention", attention(8, 4, 64, 64, 0.125, rot={"dims": 64, "base": 300.0}), 128),
        layer("attention", attention(4, 4, 128, 128, 0.09, conv=3, window=64, softcap=30.0,
                                     rot={"dims": 32, "base": 10000.0, "scaling": {"factor": 4.0, "low": 2.0, "high": 8.0, "original": 128}})),
        layer("channel_delta", delta(4, 1, 64, 64, conv=4), 64),
        layer("attention", attention(4, 4, 128, 128, 0.09, conv=2, window=200,
                                     rot={"dims": 32, "base": 10000.0, "scaling": {"factor": 4.0, "low": 2.0, "high": 8.0, "original": 128}},
                                     kv_from=2), 64),
        layer("attention", attention(4, 4, 128, 128, 0.12, softcap=10.0,
                                     rot={"dims": 32, "base": 10000.0, "scaling": {"factor": 4.0, "low": 2.0, "high": 8.0, "original": 128}},
                                     kv_from=2)),
    ],
}
# U: nothing is a multiple of 8, 4 or 2 where the design allows it; no multiplier on the logits; no rotation in
# the attention layer.
CONFIG_U = {
    "architecture": "Megerax", "vocab": 101, "width": 50, "norm": {"eps": 1e-4},
    "layers": [
        layer("channel_delta", delta(3, 3, 9, 7, conv=3), 9),
        layer("attention", attention(3, 1, 10, 5, 0.4, conv=5, window=3, softcap=2.5), 11),
        layer("latent_attention", latent(3, 5, 6, 7, 9, 5, 0.3, {"dims": 6, "base": 20.0})),
    ],
}
CONFIGS = {"P": (CONFIG_P, 3, 0.12, 0.1), "Q": (CONFIG_Q, 4, 0.08, 0.05), "U": (CONFIG_U, 5, 0.15, 0.1)}     # configuration, seed, std, norm std


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed, std, norm_std) in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"megerax_{name}"))
        lib.write_random_model(folder, cfg, seed=seed, dtype="bfloat16", std=std, norm_std=norm_std)
        out[name] = folder
    return out


_models, _weights, _memo = {}, {}, {}


def get_model(folders, name, dtype):
    if (name, dtype) not in _models:
        _models[(name, dtype)] = Model.load(folders[name], dtype=dtype, device="cuda")
    return _models[(name, dtype)]


def weights_of(folders, name):
    if name not in _weights:
        _weights[name] = plain_llama.read_safetensors(os.path.join(folders[name], "model.safetensors"))
    return _weights[name]


def want_logits(folders, name, tokens):
    key = (name, tuple(tokens))
    if key not in _memo:
        _memo[key] = plain.forward(CONFIGS[name][0], weights_of(folders, name), list(tokens))
    return _memo[key]


def prompts_of(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, CONFIGS[name][0]["vocab"], n).tolist() for n in lengths]


def t32(a):
    return torch.tensor(np.asarray(a, dtype=np.float32), device=DEV)


def f64(t):
    return t.float().cpu().numpy().astype(np.float64)


def close(got, want, dtype, what="", loose=1.0):
    lim = (2e-5 if dtype == "float32" else 2e-2) * loose
    got = f64(got) if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = np.abs(got - want)
    assert err.max() <= lim * max(1.0, np.abs(want).max()), (what, err.max(), np.unravel_index(err.argmax(), err.shape))


def run_cut(model, cache, tokens, portions):
    """Feed `tokens` in portions of the given sizes (the last size repeats), logits everywhere."""
    slot = cache.open_sequence()
    out, at, i = [], 0, 0
    while at < len(tokens):
        n = min(portions[min(i, len(portions) - 1)], len(tokens) - at)
        out.append(step(model, cache, [StepEntry(slot, tokens[at:at + n], list(range(n)))]).float().cpu().numpy())
        at += n
        i += 1
    cache.close_sequence(slot)
    return np.concatenate(out)


# ------------------------------------------------------------------ mixers alone
def mixers_of(dtype, hidden, layers, weights, eps=1e-5):
    """The mixers of a model of these layers, built by the plan and loaded with `weights`
    (names l<i>.mix.*), with a cache for them: (runtime, parts, cache)."""
    raw = {"architecture": "Megerax", "vocab": 8, "width": hidden, "norm": {"eps": eps}, "layers": layers}
    arch = find_architecture(raw)
    plan = arch.plan(arch.read_config(raw))
    rt = Runtime(DEV, TORCH[dtype])
    parts = [build_part("mixer", spec.part("mixer")) for spec in plan.layers]
    for part in parts:
        for p in walk(part):
            p.load(weights, rt)
    requests = [part.cache_requests() for part in parts]
    shared = [e.cache for e in plan.schedule]
    return rt, parts, lambda pages=6: Cache(requests, shared, max_tokens=64 * pages, max_slots=3, dtype=TORCH[dtype], device=DEV)


def run_mixers(rt, parts, cache, x, cuts, slot=None):
    """Every mixer over the same input rows, cut into steps of the given sizes."""
    slot = cache.open_sequence() if slot is None else slot
    at, got = 0, [[] for _ in parts]
    for n in cuts:
        cache.reserve_many([(slot, at + n)]); cache.flush_tables()
        ctx = context(rt, [n], [at], [slot])
        ctx.total_kv_len = at + n
        for i, part in enumerate(parts):
            got[i].append(f64(part.forward(x[at:at + n].contiguous(), ctx, cache.handles[i])))
        cache.advance(slot, n)
        at += n
    cache.close_sequence(slot)
    return [np.concatenate(g) for g in got]


def random_weights(rng, shapes, std=0.3):
    out = {}
    for name, shape in shapes.items():
        w = rng.standard_normal(shape) * std
        if name.endswith("norm"):
            w = 1 + 0.2 * rng.standard_normal(shape)
        elif name.endswith(".conv"):
            w = 1.0 / shape[1] + 0.4 * rng.standard_normal(shape)
        out[name] = t32(w).to(torch.bfloat16)
    return out


def attention_shapes(p, m, hidden, own=True):
    H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv")
    s = {p + "q": (H * d, hidden), p + "q.b": (H * d,), p + "q.norm": (d,), p + "g": (H * dv, hidden), p + "o": (hidden, H * dv)}
    if own:
        s.update({p + "k": (G * d, hidden), p + "k.b": (G * d,), p + "k.norm": (d,), p + "v": (G * dv, hidden), p + "v.b": (G * dv,)})
    if taps:
        s[p + "q.conv"] = (H * d, taps)
        if own:
            s.update({p + "k.conv": (G * d, taps), p + "v.conv": (G * dv, taps)})
    return s


def short(weights, prefix):
    return {k[len(prefix):]: f64(v) for k, v in weights.items() if k.startswith(prefix)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,window_a,window_b,dim,vdim", [(3, 1, 2, 12, 6), (2, 5, 70, 12, 6), (5, 64, 65, 12, 6), (None, 2, None, 12, 6),
                                                             (4, None, 3, 12, 6), (3, 40, 7, 8, 20), (4, 3, None, 16, 40)])
def test_attention_with_convolved_projections_short_windows_and_borrowed_keys(dtype, taps, window_a, window_b, dim, vdim):
    """Random weights, windows of 1, 2, 3 and 5 keys (every key weighs, so a window or a tap one
    off shows everywhere), a second mixer that reads the first one's keys and values through queries,
    taps, window and cap of its own; prompts against portions down to two tokens and single tokens."""
    rng = np.random.default_rng(7)
    hidden, T = 40, 150
    rot = {"dims": 6, "base": 30.0, "scaling": SCALING}
    ma = attention(4, 2, dim, vdim, 0.4, conv=taps, window=window_a, rot=rot, softcap=3.0)        # values narrower and wider than keys
    mb = attention(4, 2, dim, vdim, 0.3, conv=2, window=window_b, rot=rot, kv_from=0)
    weights = random_weights(rng, {**attention_shapes("l0.mix.", ma, hidden), **attention_shapes("l1.mix.", mb, hidden, own=False)})
    for name in ("l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l1.mix.q.b"):
        weights[name] = weights[name] * 3          # biases large enough that one added after the convolution, or to the zeros before the start, shows
    x = t32(rng.standard_normal((T, hidden))).to(TORCH[dtype])
    want_a, kv = plain.attention_mixer(f64(x), short(weights, "l0.mix."), ma, 1e-5)
    want_b, _ = plain.attention_mixer(f64(x), short(weights, "l1.mix."), mb, 1e-5, kv)
    rt, parts, new_cache = mixers_of(dtype, hidden, [layer("attention", ma), layer("attention", mb)], weights)
    assert "l1.mix.k" not in [s.name for s in parts[1].weight_specs()]
    for cuts in ([T], [1] * T, [2] * (T // 2), [63, 1, 1, 64, 21], [100] + [1] * 50, [3, 2, 145]):
        got_a, got_b = run_mixers(rt, parts, new_cache(), x, cuts)
        close(got_a, want_a, dtype, ("own", taps, window_a, cuts[:2]))
        close(got_b, want_b, dtype, ("borrowed", window_b, cuts[:2]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("needle,window", [(0, 300), (3, 1000), (63, 237), (64, 236), (64, 235), (65, 235), (127, 173), (127, 172),
                                           (128, 172), (128, 171), (290, 10), (290, 9), (299, 1), (298, 1), (150, 150), (150, 149),
                                           (0, None)])
def test_attention_finds_one_key_just_inside_its_window_and_not_just_outside(dtype, needle, window):
    """One key among 300 stands out for the last query through one channel.  The answer is half
    that token's value (the gate is sigmoid(0)) if the window reaches it (last - needle < window) and
    nothing like it if not: far keys, page borders, the window's edge, the first token; the last
    query in a prompt, alone, and after 39 decoded tokens.  Taps (0, 1) leave the projections as
    they are, so that a key is its own token's."""
    T, hidden, H, d, dv, mark = 300, 64, 2, 16, 16, 13
    m = attention(H, 1, d, dv, 1.0, conv=2, window=window, rot={"dims": 8, "base": 100.0}, softcap=50.0)
    eye, z = torch.eye(16), lambda r, c: torch.zeros(r, c)
    weights = {"q": torch.cat([torch.cat([z(16, 32), eye, z(16, 16)], dim=1)] * H), "q.b": z(H * d, 1)[:, 0],
               "k": torch.cat([eye, z(16, 48)], dim=1), "k.b": z(d, 1)[:, 0],
               "v": torch.cat([z(16, 16), eye, z(16, 32)], dim=1), "v.b": z(dv, 1)[:, 0],
               "q.norm": torch.ones(d), "k.norm": torch.ones(d), "g": z(H * dv, hidden),
               "o": torch.cat([torch.eye(32), z(32, 32)], dim=0),
               "q.conv": torch.tensor([[0.0, 1.0]] * (H * d)), "k.conv": torch.tensor([[0.0, 1.0]] * d), "v.conv": torch.tensor([[0.0, 1.0]] * dv)}
    weights = {"l0.mix." + k: v.to(torch.bfloat16) for k, v in weights.items()}
    rng = np.random.default_rng(needle)
    x = rng.standard_normal((T, hidden)) * 0.1
    x[:, mark] = 0.0
    x[needle, mark] = 9.0                                   # the key that stands out (about 4 after its norm) ...
    x[-1, 32 + mark] = 9.0                                  # ... for the last query only
    xt = t32(x).to(TORCH[dtype])
    want, _ = plain.attention_mixer(f64(xt), short(weights, "l0.mix."), m, 1e-5)
    seen = window is None or T - 1 - needle < window
    found = np.abs(want[-1, :dv] - 0.5 * f64(xt)[needle, 16:32]).max() < 0.02
    assert found == seen
    rt, parts, new_cache = mixers_of(dtype, hidden, [layer("attention", m)], weights)
    for cut in (T, T - 1, T - 40):
        got, = run_mixers(rt, parts, new_cache(), xt, [cut] + [1] * (T - cut))
        close(got, want, dtype, (needle, window, cut), loose=5.0)


def latent_shapes(p, m, hidden):
    H, d, r, dv, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    return {p + "dq": (qr, hidden), p + "dq.norm": (qr,), p + "uq": (H * (d + r), qr), p + "dkv": (rank + r, hidden),
            p + "dkv.norm": (rank,), p + "uk": (H * d, rank), p + "uv": (H * dv, rank), p + "sink": (H,), p + "o": (hidden, H * dv)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot_dim,vdim,rank,q_rank,dims,window,sink", [
    (3, 8, 4, 6, 12, 10, 4, None, 2.0), (4, 32, 16, 32, 48, 24, 16, None, -1.0), (2, 64, 32, 64, 96, 64, 16, 70, 4.0),
    (5, 5, 6, 7, 9, 5, 2, 3, 0.5), (16, 64, 64, 128, 64, 32, 64, None, 1.0)])
def test_latent_attention_with_a_query_latent_half_split_pairs_and_sinks(dtype, heads, dim, rot_dim, vdim, rank, q_rank, dims, window, sink):
    """Random weights; sinks large enough that leaving them out, scaling them or counting them twice
    (once per run of keys) shows; prompts, portions and single tokens over page borders."""
    rng = np.random.default_rng(11)
    hidden, T = 48, 200
    m = latent(heads, dim, rot_dim, vdim, rank, q_rank, 0.3, {"dims": dims, "base": 40.0}, window=window)
    weights = random_weights(rng, latent_shapes("l0.mix.", m, hidden), std=0.25)
    weights["l0.mix.sink"] = t32(sink + rng.standard_normal(heads)).to(torch.bfloat16)
    x = t32(rng.standard_normal((T, hidden))).to(TORCH[dtype])
    want = plain.latent_mixer(f64(x), short(weights, "l0.mix."), m, 1e-5)
    without = plain.latent_mixer(f64(x), dict(short(weights, "l0.mix."), sink=np.full(heads, -100.0)), m, 1e-5)
    assert np.abs(want - without).max() > 0.05 * np.abs(want).max()
    rt, parts, new_cache = mixers_of(dtype, hidden, [layer("latent_attention", m)], weights)
    for cuts in ([T], [1] * T, [2] * (T // 2), [63, 1, 1, 64, 71], [150] + [1] * 50):
        got, = run_mixers(rt, parts, new_cache(), x, cuts)
        close(got, want, dtype, (heads, dim, cuts[:2]), loose=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_finds_the_first_token_and_keys_at_page_borders(dtype):
    """One latent among 300 stands out for the last query; identity up projections return it."""
    T, hidden, heads, dim, rot_dim, rank = 300, 64, 2, 16, 8, 16
    m = latent(heads, dim, rot_dim, 16, rank, 24, 1.0, {"dims": 8, "base": 100.0})
    eye, z = torch.eye(16), lambda r, c: torch.zeros(r, c)
    weights = {"dq": torch.cat([z(24, 32), torch.eye(24), z(24, 8)], dim=1), "dq.norm": torch.ones(24),
               "uq": torch.cat([torch.eye(24)] * heads), "dkv.norm": torch.ones(16),
               "dkv": torch.cat([torch.cat([eye, z(16, 48)], dim=1), torch.cat([z(8, 16), torch.eye(8), z(8, 40)], dim=1)]),
               "uk": torch.cat([eye] * heads), "uv": torch.cat([eye] * heads), "sink": z(heads, 1)[:, 0],
               "o": torch.cat([torch.eye(32), z(32, 32)], dim=0)}
    weights = {"l0.mix." + k: v.to(torch.bfloat16) for k, v in weights.items()}
    mark = 5
    for needle in (0, 1, 63, 64, 127, 128, 255, 256, 298):
        rng = np.random.default_rng(needle)
        x = rng.standard_normal((T, hidden)) * 0.1
        x[:, mark] = 0.0
        x[needle, mark] = 9.0
        x[-1, 32 + mark] = 9.0
        xt = t32(x).to(TORCH[dtype])
        want = plain.latent_mixer(f64(xt), short(weights, "l0.mix."), m, 1e-5)
        c = plain.rms_norm(f64(xt)[:, :16], np.ones(16), 1e-5)
        assert np.abs(want[-1, :16] - c[needle]).max() < 0.05
        rt, parts, new_cache = mixers_of(dtype, hidden, [layer("latent_attention", m)], weights)
        for cut in (T, T - 1, T - 40):
            got, = run_mixers(rt, parts, new_cache(), xt, [cut] + [1] * (T - cut))
            close(got, want, dtype, (needle, cut), loose=5.0)


def delta_shapes(p, m, hidden, ranks):
    H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m.get("conv")
    s = {p + "q": (G * d, hidden), p + "k": (G * d, hidden), p + "v": (H * dv, hidden), p + "b": (H, hidden), p + "A_log": (H,),
         p + "a1": (ranks[0], hidden), p + "a2": (H * d, ranks[0]), p + "dt_bias": (H * d,), p + "g1": (ranks[1], hidden),
         p + "g2": (H * dv, ranks[1]), p + "norm": (dv,), p + "o": (hidden, H * dv)}
    if taps:
        s.update({p + "q.conv": (G * d, taps), p + "k.conv": (G * d, taps), p + "v.conv": (H * dv, taps)})
    return s


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps,ranks", [
    (4, 2, 12, 6, 3, (5, 7)), (2, 2, 64, 64, 4, (16, 8)), (6, 1, 128, 32, 2, (24, 24)), (3, 3, 9, 7, None, (3, 4)),
    (1, 1, 200, 20, 5, (8, 8)), (2, 1, 32, 130, 2, (8, 16))])
def test_the_delta_rule_carries_its_state_across_portions_and_slots(dtype, heads, kv_heads, dim, vdim, taps, ranks):
    """Random weights with decays all over (0, 1); the state and the convolution's inputs go from step
    to step through the cache; a slot that is used again starts from zero."""
    rng = np.random.default_rng(13)
    hidden, T = 40, 140
    m = delta(heads, kv_heads, dim, vdim, conv=taps)
    weights = random_weights(rng, delta_shapes("l0.mix.", m, hidden, ranks), std=0.4)
    weights["l0.mix.A_log"] = t32(rng.uniform(-3.0, 1.0, heads)).to(torch.bfloat16)
    weights["l0.mix.dt_bias"] = t32(rng.uniform(-3.0, 1.0, heads * dim)).to(torch.bfloat16)
    x = t32(rng.standard_normal((T, hidden))).to(TORCH[dtype])
    want = plain.delta_mixer(f64(x), short(weights, "l0.mix."), m, 1e-5)
    rt, parts, new_cache = mixers_of(dtype, hidden, [layer("channel_delta", m)], weights)
    cache = new_cache()
    for cuts in ([T], [1] * T, [2] * (T // 2), [63, 1, 1, 64, 11], [100] + [1] * 40, [3, 2, 135]):
        got, = run_mixers(rt, parts, cache, x, cuts)          # the same cache: every run takes a slot another run has left
        close(got, want, dtype, (heads, dim, vdim, cuts[:2]), loose=2.0)
    # two sequences side by side in one step, each against itself alone
    y = t32(rng.standard_normal((50, hidden))).to(TORCH[dtype])
    want_y = plain.delta_mixer(f64(y), short(weights, "l0.mix."), m, 1e-5)
    a, b = cache.open_sequence(), cache.open_sequence()
    got_x, got_y = [], []
    for (na, nb) in ((37, 20), (1, 1), (1, 1), (101, 28)):
        ax, ay = cache.length(a), cache.length(b)
        cache.reserve_many([(a, ax + na), (b, ay + nb)]); cache.flush_tables()
        ctx = context(rt, [na, nb], [ax, ay], [a, b])
        out = f64(parts[0].forward(torch.cat([x[ax:ax + na], y[ay:ay + nb]]).contiguous(), ctx, cache.handles[0]))
        got_x.append(out[:na]); got_y.append(out[na:])
        cache.advance(a, na); cache.advance(b, nb)
    close(np.concatenate(got_x), want, dtype, "first of two", loose=2.0)
    close(np.concatenate(got_y), want_y, dtype, "second of two", loose=2.0)


@pytest.mark.parametrize("d,n_seqs", [(64, 37), (64, 19), (64, 10), (64, 2), (128, 19), (128, 10), (128, 3), (256, 10), (256, 2),
                                      (96, 3), (16, 40)])
def test_the_recurrence_kernels_for_every_split_of_the_state(d, n_seqs):
    """The recurrence alone, for every number of lanes that share a column of the state (the launcher picks it
    by how many columns a step brings): unequal sequences in one step, a second step that continues them, then a
    step of one token each; every sequence against the plain recurrence, head by head."""
    rng = np.random.default_rng(d + n_seqs)
    H, G, dv = 8, 4, 64
    lens = [[1 + (b + k) % 5 for b in range(n_seqs)] for k in range(2)] + [[1] * n_seqs]
    total = [sum(l[b] for l in lens) for b in range(n_seqs)]
    q = rng.standard_normal((n_seqs, max(total), G, d)); q /= np.linalg.norm(q, axis=-1, keepdims=True) * np.sqrt(d)
    k = rng.standard_normal((n_seqs, max(total), G, d)); k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.standard_normal((n_seqs, max(total), H, dv))
    g = rng.uniform(0.05, 1.0, (n_seqs, max(total), H, d))
    beta = rng.uniform(0.0, 1.0, (n_seqs, max(total), H))
    state = torch.zeros(n_seqs + 1, H, d, dv, dtype=torch.float32, device=DEV)
    slots = torch.tensor([n_seqs - b for b in range(n_seqs)], dtype=torch.int32, device=DEV)       # not in order, slot 0 unused
    got = [[] for _ in range(n_seqs)]
    at = [0] * n_seqs
    for step_lens in lens:
        rows = lambda a, width: np.concatenate([a[b, at[b]:at[b] + step_lens[b]].reshape(step_lens[b], width) for b in range(n_seqs)])
        qk = t32(np.concatenate([rows(q, G * d), rows(k, G * d)], axis=1))
        vt, gt, bt = t32(rows(v, H * dv)), t32(rows(g, H * d)), t32(rows(beta, H))
        out = torch.empty(sum(step_lens), H * dv, dtype=torch.float32, device=DEV)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(step_lens)]), dtype=torch.int32, device=DEV)
        ops.delta_scan(qk, vt, gt, bt, state, out, cu, slots, n_seqs, H, G, d, dv, one_token_each=max(step_lens) == 1)
        o = f64(out)
        for b in range(n_seqs):
            got[b].append(o[int(cu[b]):int(cu[b + 1])])
            at[b] += step_lens[b]
    for b in range(0, n_seqs, max(1, n_seqs // 4)):
        T = total[b]
        f = lambda a: f64(t32(a))
        for h in range(H):
            want = plain.delta_rule(f(q[b, :T, h // 2]), f(k[b, :T, h // 2]), f(v[b, :T, h]), f(beta[b, :T, h]), f(g[b, :T, h]))
            close(np.concatenate(got[b])[:, h * dv:(h + 1) * dv], want, "float32", (d, n_seqs, b, h), loose=2.0)
    assert float(state[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_delta_rule_remembers_its_first_token_where_it_does_not_decay(dtype):
    """Head 0 forgets almost nothing (a rate of e^-12), head 1 forgets within a few tokens.  The first
    token writes a value that stands out along a key that only the last query asks for again: 149
    tokens later head 0 still returns it and head 1 does not."""
    T, hidden, d, dv = 150, 64, 16, 16
    m = delta(2, 2, d, dv, conv=2)
    eye, z = torch.eye(16), lambda r, c: torch.zeros(r, c)
    pick = lambda at: torch.cat([z(16, at), eye, z(16, hidden - at - 16)], dim=1)
    weights = {"q": torch.cat([pick(0)] * 2), "k": torch.cat([pick(0)] * 2), "v": torch.cat([pick(16)] * 2), "b": z(2, hidden),
               "A_log": torch.tensor([-12.0, 1.0]), "a1": z(4, hidden), "a2": z(2 * d, 4), "dt_bias": z(2 * d, 1)[:, 0],
               "g1": z(4, hidden), "g2": z(2 * dv, 4), "norm": torch.ones(dv), "o": torch.cat([torch.eye(32), z(32, 32)], dim=0),
               "q.conv": torch.tensor([[0.0, 1.0]] * (2 * d)), "k.conv": torch.tensor([[0.0, 1.0]] * (2 * d)),
               "v.conv": torch.tensor([[0.0, 1.0]] * (2 * dv))}
    weights["b"][:, 63] = 4.0                                # beta = sigmoid(4 x_63)
    weights = {"l0.mix." + k: v.to(torch.bfloat16) for k, v in weights.items()}
    rng = np.random.default_rng(2)
    x = rng.standard_normal((T, hidden)) * 0.05
    x[:, 5] = 0.0                                            # no later key has anything of channel 5 ...
    x[0, 5] = x[-1, 5] = 6.0                                 # ... but the first token's, and the last query asks for it
    x[:, 63] = 1.0
    x[-1, 63] = -2.0                                         # the last token itself writes next to nothing (beta = sigmoid(-8))
    x[0, 16:32] = np.linspace(2.0, 5.0, 16)                  # the value that stands out
    xt = t32(x).to(TORCH[dtype])
    want = plain.delta_mixer(f64(xt), short(weights, "l0.mix."), m, 1e-5)
    first = plain.silu(f64(xt)[0, 16:32])
    shape = lambda v: v / np.sqrt((v * v).mean())
    assert np.abs(shape(want[-1, :dv]) - shape(first)).max() < 0.1          # head 0: the first token's value, normed
    assert np.abs(shape(want[-1, dv:2 * dv]) - shape(first)).max() > 0.5     # head 1 has long forgotten it
    rt, parts, new_cache = mixers_of(dtype, hidden, [layer("channel_delta", m)], weights)
    for cuts in ([T], [T - 1, 1], [1] * T, [2] * (T // 2), [64, 64, 22]):
        got, = run_mixers(rt, parts, new_cache(), xt, cuts)
        close(got, want, dtype, cuts[:2], loose=3.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_feed_forward_with_the_tanh_form_of_gelu(dtype):
    rng = np.random.default_rng(6)
    for n, hidden, ff in [(1, 16, 8), (70, 72, 100), (200, 128, 264), (17, 50, 11)]:
        names = {"gate": (ff, hidden), "up": (ff, hidden), "down": (hidden, ff)}
        w = {k: (t32(rng.standard_normal(s)) * 0.5).to(torch.bfloat16) for k, s in names.items()}
        part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": ff, "activation": "gelu_tanh",
                                                              "gate": "gate", "up": "up", "down": "down"}))
        rt = Runtime(DEV, TORCH[dtype])
        part.load(w, rt)
        x = t32(rng.standard_normal((n, hidden))).to(TORCH[dtype])
        got = part.forward(x, context(rt, [n], [0], [0]))
        want = plain.gated_feed_forward(f64(x), f64(w["gate"]), f64(w["up"]), f64(w["down"]))
        close(got, want, dtype, (n, hidden, ff), loose=2.0)
        silu_part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": ff,
                                                                   "gate": "gate", "up": "up", "down": "down"}))
        silu_part.load(w, rt)
        other = f64(silu_part.forward(x, context(rt, [n], [0], [0])))
        assert np.abs(other - want).max() > 1e-3 * np.abs(want).max()      # the activation is not silu's


def test_the_norm_behind_the_embedding_and_the_multiplier_on_the_logits():
    rng = np.random.default_rng(3)
    for n, h in [(1, 8), (5, 72), (70, 1000), (3, 4100)]:
        x, w = rng.standard_normal((n, h)) * 3, 1 + 0.2 * rng.standard_normal(h)
        xt, wt = t32(x), t32(w)
        ops.rmsnorm_rows(xt, wt, 1e-3)
        close(xt, plain.rms_norm(f64(t32(x)), f64(wt), 1e-3), "float32", (n, h))
        ops.scale(xt, 0.37)
        close(xt, 0.37 * plain.rms_norm(f64(t32(x)), f64(wt), 1e-3), "float32", (n, h))


# ------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "U"])
def test_whole_prompts_of_many_lengths_and_the_hidden_state_after_every_layer(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    for p in prompts_of(name, [1, 2, 3, 17, 63, 64, 65, 129, 230]):
        got = run_cut(model, cache, p, [len(p)])
        assert_close(got, want_logits(folders, name, p), dtype, f"{name} {dtype} whole prompt of {len(p)}")
    assert cache.open_slots() == []
    p = prompts_of(name, [90], seed=3)[0]
    hidden, layers = [], []
    model.op_hook = lambda s, l, op, t: hidden.append(f64(t)) if op == "hidden_post_ffn" else None
    try:
        run_cut(model, cache, p, [len(p)])
    finally:
        model.op_hook = None
    plain.forward(CONFIGS[name][0], weights_of(folders, name), p, layers_out=layers)
    assert len(hidden) == len(layers)
    for i, (g, w) in enumerate(zip(hidden, layers)):
        close(g, w, dtype, f"{name} {dtype} hidden state after layer {i}", loose=4.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "U"])
def test_portions_down_to_two_tokens_and_token_by_token_from_the_start(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    p = prompts_of(name, [150], seed=5)[0]
    want = want_logits(folders, name, p)
    rows = {}
    for portions in ([150], [1], [2], [3, 2, 1, 16, 15, 17, 64], [63, 1, 1, 64, 2], [100, 1]):
        rows[tuple(portions)] = run_cut(model, cache, p, portions)
        assert_close(rows[tuple(portions)], want, dtype, f"{name} {dtype} portions {portions}")
    if dtype == "float32":
        # sums walk keys, taps and channels in one order whatever the cut
        for portions, got in rows.items():
            np.testing.assert_allclose(got, rows[(150,)], rtol=0, atol=2e-5 * np.abs(want).max(), err_msg=str(portions))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "U"])
def test_long_decoding_across_page_borders_and_windows(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    p = prompts_of(name, [5 + 280], seed=6)[0]
    got = run_cut(model, cache, p, [5, 1])
    assert_close(got, want_logits(folders, name, p), dtype, f"{name} {dtype} 280 tokens decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_unequal_batches_against_each_alone_with_slots_and_pages_used_again(folders, name, dtype):
    """Three batches through a cache too small for two of them: the slots and pages
    of finished requests, with their old rows and states, go to new ones.  In a batch every
    request is decoded to its own length and leaves when it ends."""
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 7, max_slots=4)
    batches = [[(5, 9), (70, 3), (17, 20), (1, 12)], [(64, 1), (130, 6), (3, 33)], [(40, 8), (128, 2), (9, 9), (2, 2)]]
    for bi, batch in enumerate(batches):
        prompts = prompts_of(name, [a + b for a, b in batch], seed=20 + bi)
        slots = [cache.open_sequence() for _ in batch]
        got = [[] for _ in batch]
        entries = [StepEntry(slots[i], p[:plen], list(range(plen))) for i, ((plen, _), p) in enumerate(zip(batch, prompts))]
        flat = step(model, cache, entries).float().cpu().numpy()
        o = 0
        for i, e in enumerate(entries):
            got[i].append(flat[o:o + len(e.want)])
            o += len(e.want)
        live, t = list(range(len(batch))), 0
        while True:
            live = [i for i in live if t < batch[i][1]]
            if not live:
                break
            flat = step(model, cache, [StepEntry(slots[i], [prompts[i][batch[i][0] + t]], [0]) for i in live]).float().cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(flat[j:j + 1])
                if t + 1 >= batch[i][1]:
                    cache.close_sequence(slots[i])
            t += 1
        for i in range(len(batch)):
            assert_close(np.concatenate(got[i]), want_logits(folders, name, prompts[i]), dtype, f"{name} {dtype} batch {bi} request {i}")
        assert cache.open_slots() == []
    assert all(free == 7 for free in cache.free_pages())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype):
    model = get_model(folders, name, dtype)
    assert model.capturable
    prompts = prompts_of(name, [5, 17, 40, 1], seed=7)
    cfg, w = CONFIGS[name][0], weights_of(folders, name)
    for use_graph in (True, False):
        results = lib.generate(model, prompts, [12, 6, 9, 12], stop=[], use_graph=use_graph)
        assert [len(r.tokens) for r in results] == [12, 6, 9, 12]
        ok = []
        for p, r in zip(prompts, results):
            seq = list(p)
            for tok in r.tokens:                          # each token is one the plain model could have chosen there
                logits = plain.forward(cfg, w, seq)[-1]
                slack = (1e-4 if dtype == "float32" else 5e-2) * max(1.0, np.abs(logits).max())
                ok.append(logits[tok] >= logits.max() - slack)
                seq.append(tok)
        assert all(ok), (use_graph, ok)
    if dtype == "float32":
        assert results[1].tokens == plain.greedy(cfg, w, prompts[1], 6)


def test_trace_replay_and_command_line(folders, tmp_path):
    """bin/trace_run with a batch that starts together and shrinks, and llmgen with token ids."""
    name = "P"
    a, b = prompts_of(name, [30, 9], seed=8)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:20], "want": [0, 19]}, {"id": "y", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[20:21], "want": [0]}, {"id": "y", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[21:22], "want": []}, {"id": "y", "tokens": b[8:9], "want": [0]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": a[22:], "want": [7]}], "end": ["x"]}]
    out = str(tmp_path / "out")
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name], "--dtype", "float32",
                           "--out", out, "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wb = want_logits(folders, name, a), want_logits(folders, name, b)
    V = CONFIGS[name][0]["vocab"]
    read = lambda i: np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, V)
    assert_close(read(0), np.stack([wa[0], wa[19], wb[6]]), "float32", "step 0")
    assert_close(read(1), wa[20:21], "float32", "step 1")
    assert_close(read(2), wb[8:9], "float32", "step 2")
    assert_close(read(3), wa[29:30], "float32", "step 3")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmgen"), "-model", folders[name], "-ids",
                           ",".join(str(t) for t in b), "-tokens", "5", "-dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    want = plain.greedy(CONFIGS[name][0], weights_of(folders, name), b, 5)
    assert " ".join(str(t) for t in want) in proc.stdout.replace(",", " ").replace("[", " ").replace("]", " ")
