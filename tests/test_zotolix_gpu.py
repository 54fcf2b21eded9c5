"""The Zotolix design in the engine against its plain implementation
(plain_zotolix.py): every mechanism alone, then whole models of three small
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
import plain_zotolix as plain
from go_tinygrad_b200.cache import Cache, KVRequest
from go_tinygrad_b200.engine import Model, StepEntry, step
from go_tinygrad_b200.kernels import ops
from go_tinygrad_b200.parts import PartSpec, Runtime, build_part, walk
from conftest import ROOT, assert_close
from test_parts_gpu import context
from test_senupel_gpu import Choices, close, f64, join, t32
from test_zotolix_config import mixer as mixer_json, moe

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda" if torch.cuda.is_available() and torch.cuda.device_count() else "cpu")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


# R: three copies; values wider than keys; a head of 20 channels (no multiple of 8: the plain attention kernel in
# both dtypes) beside heads the tensor-core kernel takes; stretches shorter than a page, of exactly a page and longer
# than anything fed; a layer that blends nothing between layers that do; a layer without a feed-forward; part of a head
# rotating and all of it; one expert of four, two of five, all three of three.
CONFIG_R = {
    "architecture": "Zotolix", "vocab": 211, "width": 72, "norm": {"eps": 1e-4}, "embedding": {"scale": 3.0},
    "residual_mult": 0.7, "streams": 3,
    "layers": [
        layer("attention_2", mixer_json(6, 2, 24, 40, 70, 0.2, 16, 100.0, v_mix=True), moe(36, 5, 2)),
        layer("attention", mixer_json(3, 3, 20, 12, 33, 0.3, 10, 1000.0), None),
        layer("attention", mixer_json(4, 2, 16, 40, 64, 0.25, 16, 50.0, v_mix=True), moe(20, 3, 3)),
        layer("attention_2", mixer_json(2, 2, 32, 40, 1000, 0.17, 8, 1000.0, v_mix=True), moe(24, 4, 1)),
    ],
}
# S: no copies and no multipliers at all (the ordinary residual sum, unscaled embedding); heads of 128 and 64 channels
# with values of 64 and 128; one key/value head for eight query heads and one for each; a stretch of 5 keys and one of
# 150; the first layer blends nothing, so the second is the one whose values the third takes.
CONFIG_S = {
    "architecture": "Zotolix", "vocab": 160, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention", mixer_json(8, 1, 128, 64, 150, 0.09, 64, 10000.0), moe(64, 8, 2)),
        layer("attention_2", mixer_json(4, 4, 64, 128, 64, 0.125, 32, 300.0, v_mix=True), moe(32, 2, 2)),
        layer("attention_2", mixer_json(16, 4, 64, 128, 5, 0.2, 64, 77.0, v_mix=True), None),
        layer("attention", mixer_json(2, 1, 64, 8, None, 0.15, 2, 10000.0), moe(264, 3, 1)),
    ],
}
# U: one copy with links of its own; nothing is a multiple of 8, 4 or 2 where the design allows it.
CONFIG_U = {
    "architecture": "Zotolix", "vocab": 101, "width": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
    "residual_mult": 1.3, "streams": 1,
    "layers": [
        layer("attention", mixer_json(3, 3, 7, 5, 3, 0.4, 4, 20.0, v_mix=True), moe(9, 3, 2)),
        layer("attention_2", mixer_json(3, 3, 5, 5, 70, 0.3, 2, 20.0, v_mix=True), moe(11, 2, 1)),
    ],
}
CONFIGS = {"R": (CONFIG_R, 3, 0.12, 0.1), "S": (CONFIG_S, 4, 0.08, 0.05), "U": (CONFIG_U, 5, 0.15, 0.1)}     # configuration, seed, std, norm std


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed, std, norm_std) in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"zotolix_{name}"))
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


def model_close(folders, name, dtype, tokens, got, routing, what):
    if dtype == "float32":
        want = want_logits(folders, name, tokens)
        own = plain.forward(CONFIGS[name][0], weights_of(folders, name), list(tokens), experts_of=routing)
        assert np.array_equal(own, want), f"{what}: the model chose other experts than the plain implementation"
        return assert_close(got, want, dtype, what)
    # bfloat16: the plain implementation follows the model's expert choices (two router scores may be
    # closer than the rounding of the router's input).  A wrong key or stretch errs by about 1.
    want = plain.forward(CONFIGS[name][0], weights_of(folders, name), list(tokens), experts_of=routing)
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    scale, err = max(1.0, float(np.abs(want).max())), np.abs(got - want)
    assert err.mean() <= 6e-3 * scale, f"{what}: mean error {err.mean():.3e}"
    assert err.max() <= 8e-2 * scale, f"{what}: max error {err.max():.3e} at {np.unravel_index(int(err.argmax()), err.shape)}"


def run_cut(model, cache, tokens, portions):
    """Feed `tokens` in portions of the given sizes (the last size repeats), logits everywhere.
    Returns (logits, {layer: the experts every token used})."""
    listen = Choices(model)
    slot = cache.open_sequence()
    out, used, at, i = [], [], 0, 0
    while at < len(tokens):
        n = min(portions[min(i, len(portions) - 1)], len(tokens) - at)
        out.append(step(model, cache, [StepEntry(slot, tokens[at:at + n], list(range(n)))]).float().cpu().numpy())
        used += listen.take([n])
        at += n
        i += 1
    cache.close_sequence(slot)
    listen.close()
    return np.concatenate(out), join(used)


# ---------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S,H,n", [(1, 48, 7), (3, 50, 33), (4, 256, 70), (8, 1024, 5), (2, 13000, 3)])
def test_copies_of_the_hidden_state_are_made_updated_read_and_normed(dtype, S, H, n):
    rng = np.random.default_rng(S * 100 + n)
    seed, w = rng.standard_normal((n, H)), 1.0 + 0.2 * rng.standard_normal(H)
    links = [(rng.standard_normal(S), np.eye(S) + 0.3 * rng.standard_normal((S, S)), rng.standard_normal(S)) for _ in range(3)]
    copies = torch.empty(n, S, H, dtype=torch.float32, device=DEV)
    out = torch.empty(n, H, dtype=TORCH[dtype], device=DEV)
    ops.hyper_norm(copies, t32(w), 1e-5, out, seed=t32(seed), in_w=t32(links[0][0]))
    xs = np.stack([seed] * S)
    close(out, plain.rms_norm(plain.streams_read(xs, links[0][0]), w, 1e-5), dtype, "made from the seed")
    np.testing.assert_allclose(f64(copies).transpose(1, 0, 2), xs, rtol=1e-6, atol=1e-6)
    for q, float_update in ((1, False), (2, True)):
        y = rng.standard_normal((n, H))
        yt = t32(y) if float_update else t32(y).to(TORCH[dtype])
        y = f64(yt)
        in_w, (_, mix, out_w) = links[q][0], links[q - 1]
        ops.hyper_norm(copies, t32(w), 1e-5, out, update=yt, mix=t32(mix), out_w=t32(out_w), in_w=t32(in_w))
        xs = plain.streams_write(xs, y, mix, out_w, 1.0)
        close(out, plain.rms_norm(plain.streams_read(xs, in_w), w, 1e-5), dtype, f"sublayer {q}")
        np.testing.assert_allclose(f64(copies).transpose(1, 0, 2), xs, rtol=1e-5, atol=1e-5 * np.abs(xs).max())
    # the final norm: chosen rows, the plain sum of the copies, a pending update applied on the way, nothing written
    rows = [n - 1, 0, n // 2]
    y = rng.standard_normal((n, H))
    before = copies.clone()
    out = torch.empty(len(rows), H, dtype=TORCH[dtype], device=DEV)
    ops.hyper_norm(copies, t32(w), 1e-5, out, update=t32(y), mix=t32(links[2][1]), out_w=t32(links[2][2]),
                   rows=torch.tensor(rows, dtype=torch.int32, device=DEV))
    new = plain.streams_write(xs, y, links[2][1], links[2][2], 1.0)
    close(out, plain.rms_norm(new.sum(axis=0)[rows], w, 1e-5), dtype, "final norm on chosen rows")
    assert torch.equal(before, copies)


def _finish(dtype, n_heads, n_kv, hd, vd, rot, base, starts, lens, *, unit, gate, blend, seed=0, chunk=50):
    """Float sums of a projection through `qkv_finish` into a cache, the rows cut into one sequence per
    (start, length); returns what the plain pieces say and what the kernel left."""
    rng = np.random.default_rng(seed)
    n = sum(lens)
    width = n_heads * hd + n_kv * (hd + vd) + (n_heads if gate else 0)
    sums = rng.standard_normal((n, width + 3))                  # wider rows than needed: a stride of their own
    bias = rng.standard_normal(width - (n_heads if gate else 0))
    v_first = rng.standard_normal((n, n_kv * vd))
    rt = Runtime(DEV, TORCH[dtype])
    cache = Cache([[KVRequest(n_kv, hd, None, value_dim=vd, chunk=chunk)]], [None],
                  max_tokens=max(64 * 8, 64 * sum((a + l + 63) // 64 for a, l in zip(starts, lens))), max_slots=len(lens) + 1,
                  dtype=TORCH[dtype], device=DEV)
    cache.open_sequence()                                       # slot 0 stays unused: slots and batch places differ
    slots = [cache.open_sequence() for _ in lens]
    cache.reserve_many([(s, a + l) for s, a, l in zip(slots, starts, lens)]); cache.flush_tables()
    ctx = context(rt, lens, starts, slots)
    table = None
    if rot:
        position = build_part("position", PartSpec("rotary", {"head_dim": hd, "rotary_dim": rot, "theta": base}))
        position.load({}, rt)
        table = position.rotation(ctx)
    kv = cache.handles[0].kv
    q_out = torch.zeros(n, n_heads * hd + 8, dtype=TORCH[dtype], device=DEV)
    gate_out = torch.zeros(n, n_heads, dtype=torch.float32, device=DEV) if gate else None
    v_keep = torch.zeros(n, n_kv * vd, dtype=torch.float32, device=DEV)
    ops.qkv_finish(t32(sums), t32(bias), table, n_heads, kv, q_out, ctx.token_seq, ctx.slots, ctx.positions, unit_norm=unit, eps=1e-3,
                   v_first=t32(v_first) if blend is not None else None, v_keep=v_keep, blend=blend or 0.0, gate_out=gate_out)
    pos = np.concatenate([np.arange(a, a + l) for a, l in zip(starts, lens)])
    sums32, bias32, vf32 = f64(t32(sums)), f64(t32(bias)), f64(t32(v_first))
    x = sums32[:, :bias32.shape[0]] + bias32
    q = x[:, :n_heads * hd].reshape(n, n_heads, hd)
    k = x[:, n_heads * hd:n_heads * hd + n_kv * hd].reshape(n, n_kv, hd)
    v = x[:, n_heads * hd + n_kv * hd:].reshape(n, n_kv, vd)
    if rot:
        q, k = plain.rotate_heads(q, pos, rot, base), plain.rotate_heads(k, pos, rot, base)
    if unit:
        q, k = plain.unit_rms(q, 1e-3), plain.unit_rms(k, 1e-3)
    close(v_keep, v.reshape(n, -1), "float32", "values kept unblended")
    if blend is not None:
        v = plain.blend_values(v, vf32.reshape(n, n_kv, vd), np.float32(blend))
    close(q_out[:, :n_heads * hd], q.reshape(n, -1), dtype, "queries")
    assert (q_out[:, n_heads * hd:] == 0).all()
    if gate:
        close(gate_out, plain.sigmoid(sums32[:, width - n_heads:width]), "float32", "gate")
    at = 0
    for s, a, l in zip(slots, starts, lens):
        for j in range(l):
            p = a + j
            page = cache.groups[0].pages_of[s][p // 64]
            close(kv.k[page, :, p % 64], k[at + j], dtype, f"key of position {p}")
            close(kv.v[page, :, p % 64], v[at + j], dtype, f"value of position {p}")
        at += l


@pytest.mark.parametrize("dtype", DTYPES)
def test_projection_sums_are_biased_rotated_normed_blended_gated_and_stored(dtype):
    _finish(dtype, 4, 2, 16, 24, 8, 100.0, [0, 60], [70, 9], unit=True, gate=False, blend=0.4)
    _finish(dtype, 6, 3, 10, 5, 10, 50.0, [126, 0, 63], [3, 1, 2], unit=False, gate=True, blend=None, seed=1)
    _finish(dtype, 2, 1, 128, 64, 64, 1e6, [200], [1], unit=True, gate=True, blend=1.0, seed=2)
    _finish(dtype, 1, 1, 6, 7, 0, 1.0, [5], [4], unit=False, gate=False, blend=0.0, seed=3)
    # many tokens take the kernel with a block a token, few the one with a warp a head: the same numbers from both
    _finish(dtype, 5, 1, 24, 16, 12, 300.0, [0, 3], [530, 70], unit=True, gate=True, blend=0.25, seed=4, chunk=None)
    _finish(dtype, 3, 3, 9, 5, 4, 30.0, [7], [520], unit=False, gate=False, blend=None, seed=5, chunk=None)


def _filled_cache(dtype, n_kv, hd, vd, lengths, rng, chunk=None, window=None):
    """A cache whose sequences hold random keys and values for `lengths` tokens."""
    cache = Cache([[KVRequest(n_kv, hd, window, value_dim=vd, chunk=chunk)]], [None], max_tokens=64 * 24, max_slots=len(lengths) + 1,
                  dtype=TORCH[dtype], device=DEV)
    cache.open_sequence()
    kv = cache.handles[0].kv
    slots, ks, vs = [], [], []
    for L in lengths:
        s = cache.open_sequence()
        cache.reserve(s, L)
        k, v = rng.standard_normal((L, n_kv, hd)), rng.standard_normal((L, n_kv, vd))
        kt, vt = t32(k).to(TORCH[dtype]), t32(v).to(TORCH[dtype])
        for p in range(L):
            page = cache.groups[0].pages_of[s][p // 64]
            kv.k[page, :, p % 64] = kt[p]
            kv.v[page, :, p % 64] = vt[p]
        slots.append(s); ks.append(f64(kt)); vs.append(f64(vt))
    cache.flush_tables()
    return cache, kv, slots, ks, vs


def _plain_rows(q, k, v, start, scale, chunk, window):
    """Attention of the rows q [n, H, d] at positions start.. over keys 0..start+n-1."""
    n = q.shape[0]
    full = np.zeros((start + n,) + q.shape[1:])
    full[start:] = q
    if window:
        # a window beside stretches: mask by hand through very negative keys is not possible; use the visible set
        out = np.zeros((n, q.shape[1], v.shape[2]))
        G = k.shape[1]
        for i in range(n):
            p = start + i
            lo = max(0, p - window + 1)
            if chunk:
                lo = max(lo, p - p % chunk)
            for h in range(q.shape[1]):
                g = h // (q.shape[1] // G)
                s = (k[lo:p + 1, g] @ q[i, h]) * scale
                w = np.exp(s - s.max())
                out[i, h] = (w / w.sum()) @ v[lo:p + 1, g]
        return out
    return plain.attend(full, k, v, scale, chunk)[start:]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,vd", [(6, 3, 128, 56), (8, 1, 64, 128), (3, 3, 24, 40), (6, 2, 16, 8), (2, 2, 128, 128),
                                                  (5, 5, 20, 12), (12, 4, 8, 72), (8, 2, 64, 64)])
@pytest.mark.parametrize("chunk,window", [(None, None), (1, None), (5, None), (64, None), (70, None), (200, None), (1000, None),
                                          (None, 70), (100, 33)])
def test_attention_over_stretches_of_keys_in_prompts_portions_and_decode_steps(dtype, heads, kv_heads, hd, vd, chunk, window):
    rng = np.random.default_rng(heads * 1000 + hd + (chunk or 0))
    # what each sequence brings after what it holds: whole prompts, portions that start inside a page and a
    # stretch, single tokens, all in one batch
    starts, lens = [0, 0, 61, 199, 200, 330, 64], [1, 150, 90, 1, 1, 70, 2]
    cache, kv, slots, ks, vs = _filled_cache(dtype, kv_heads, hd, vd, [a + l for a, l in zip(starts, lens)], rng, chunk, window)
    rt = Runtime(DEV, TORCH[dtype])
    n = sum(lens)
    q = t32(rng.standard_normal((n, heads * hd)) * 1.5).to(TORCH[dtype])
    gate = torch.rand(n, heads, dtype=torch.float32, device=DEV)
    scale = 0.7 / np.sqrt(hd)
    want, at = [], 0
    for b, (a, l) in enumerate(zip(starts, lens)):
        o = _plain_rows(f64(q[at:at + l]).reshape(l, heads, hd), ks[b], vs[b], a, scale, chunk, window)
        want.append(o * f64(gate[at:at + l])[:, :, None])
        at += l
    want = np.concatenate(want).reshape(n, heads * vd)
    ctx = context(rt, lens, starts, slots)
    out = torch.zeros(n, heads * vd, dtype=TORCH[dtype], device=DEV)
    ops.attention_general(q, out, kv, ctx, heads, scale, window=window or 0, chunk=chunk or 0, gate=gate)
    close(out, want, dtype, "one batch of prompts, portions and single tokens")
    if dtype == "bfloat16" and ops.attention_masked_supports(kv):
        for splits in (2, 3, 7):
            scratch = torch.empty(n * heads * splits * 130, dtype=torch.float32, device=DEV)
            out.zero_()
            ops.attention_masked_bf16(q, out, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos, ctx.n_seqs, ctx.max_q_len, heads, scale,
                                      window or 0, chunk or 0, gate, splits, scratch)
            close(out, want, dtype, f"the pages cut into {splits} shares")
    else:
        assert dtype == "float32" or hd % 8 or vd % 8
    assert ops.bounded_wait_failures() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("needle,chunk,query", [(0, 300, 299), (0, 300, 300), (3, 1000, 400), (63, 64, 64), (64, 64, 127), (64, 64, 128),
                                                (128, 64, 191), (199, 200, 200), (200, 200, 399), (200, 200, 400), (255, 128, 256),
                                                (256, 128, 383), (100, 7, 104), (100, 7, 105), (98, 7, 104), (97, 7, 98)])
def test_attention_finds_one_key_just_inside_its_stretch_and_not_just_outside(dtype, needle, chunk, query):
    """One key among hundreds is made to stand out (a long key in a direction the query shares) and its value
    marked.  The token at `query` sees it exactly when both lie in one stretch: as a row of a whole
    prompt, of a portion, and decoded alone after the cache was filled through the finishing kernel."""
    heads, n_kv, hd, vd = 4, 2, 32, 16
    rng = np.random.default_rng(needle * 7 + chunk)
    total = query + 3
    width = heads * hd + n_kv * (hd + vd)
    sums = rng.standard_normal((total, width)) * 0.3
    direction = rng.standard_normal(hd)
    direction /= np.linalg.norm(direction)
    k0, v0 = heads * hd, heads * hd + n_kv * hd
    sums[needle, k0:k0 + n_kv * hd] = np.tile(direction * 40.0, n_kv)
    sums[needle, v0:v0 + n_kv * vd] = 100.0
    sums[query, :heads * hd] = np.tile(direction * 3.0, heads)
    seen = needle <= query and needle // chunk == query // chunk
    for cuts in ([total], [query, 1, 2], [needle + 1, query - needle - 1, 1, 1, 1] if query > needle + 1 else [total]):
        cuts = [c for c in cuts if c > 0]
        rt = Runtime(DEV, TORCH[dtype])
        cache = Cache([[KVRequest(n_kv, hd, None, value_dim=vd, chunk=chunk)]], [None], max_tokens=64 * 8, max_slots=2,
                      dtype=TORCH[dtype], device=DEV)
        slot = cache.open_sequence()
        kv = cache.handles[0].kv
        at, rows = 0, []
        for c in cuts:
            cache.reserve(slot, at + c); cache.flush_tables()
            ctx = context(rt, [c], [at], [slot])
            q = torch.empty(c, heads * hd, dtype=TORCH[dtype], device=DEV)
            ops.qkv_finish(t32(sums[at:at + c]), None, None, heads, kv, q, ctx.token_seq, ctx.slots, ctx.positions)
            out = torch.empty(c, heads * vd, dtype=TORCH[dtype], device=DEV)
            ops.attention_general(q, out, kv, ctx, heads, 1.0, chunk=chunk)
            rows.append(f64(out))
            cache.advance(slot, c)
            at += c
        got = np.concatenate(rows)[query]
        if seen:
            assert got.min() > 99.0, (cuts, got.min())
        else:
            assert np.abs(got).max() < 5.0, (cuts, np.abs(got).max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,hidden,ff,n", [(5, 1, 48, 20, 150), (3, 3, 48, 24, 150), (12, 4, 50, 21, 150),
                                                     (40, 2, 64, 16, 33), (2, 1, 128, 64, 700), (8, 2, 256, 128, 1)])
def test_experts_scored_by_sigmoids_take_scaled_inputs_and_add_up(dtype, experts, top, hidden, ff, n):
    rng = np.random.default_rng(experts * 10 + top)
    w = {"router": rng.standard_normal((experts, hidden)) * 0.3}
    for e in range(experts):
        w[f"e{e}.up"], w[f"e{e}.down"] = rng.standard_normal((ff, hidden)) * 0.15, rng.standard_normal((hidden, ff)) * 0.15
    tensors = {k: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for k, v in w.items()}
    w = {k: f64(v) for k, v in tensors.items()}
    spec = PartSpec("routed_experts", {"hidden_size": hidden, "intermediate_size": ff, "n_experts": experts, "top": top,
                                       "router": "router", "gate": None, "up": "e{e}.up", "down": "e{e}.down",
                                       "activation": "relu2", "scoring": "sigmoid", "weight_on": "input"})
    rt = Runtime(DEV, TORCH[dtype])
    part = build_part("feed_forward", spec)
    part.load(tensors, rt)
    x = t32(rng.standard_normal((n, hidden))).to(TORCH[dtype])
    ctx = context(rt, [n], [0], [0])
    chosen = {}
    ctx.op_hook = lambda s, l, op, t: chosen.__setitem__(op, t.cpu().numpy().copy()) if op == "experts" else None
    for float_updates in (False, True):
        ctx.float_updates = float_updates
        got = part.forward(x, ctx)
        assert got.dtype == (torch.float32 if float_updates else TORCH[dtype])
        ups, downs = [w[f"e{e}.up"] for e in range(experts)], [w[f"e{e}.down"] for e in range(experts)]
        idx, _ = plain.choose_experts(f64(x), w["router"], top)
        if dtype == "float32":
            assert np.array_equal(idx, chosen["experts"])
        else:
            assert (np.sort(idx, -1) == np.sort(chosen["experts"], -1)).mean() > 0.97
        want = plain.mixture(f64(x), w["router"], ups, downs, top, chosen=chosen["experts"])
        close(got, want, dtype, f"{top} of {experts} experts")


# ---------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R", "S", "U"])
def test_whole_prompts_of_many_lengths(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    for p in prompts_of(name, [1, 2, 3, 17, 63, 64, 65, 129, 230]):
        got, used = run_cut(model, cache, p, [len(p)])
        model_close(folders, name, dtype, p, got, used, f"{name} {dtype} whole prompt of {len(p)}")
    assert cache.open_slots() == []


@pytest.mark.parametrize("dtype", DTYPES)
def test_hidden_state_after_every_layer(folders, dtype):
    name = "R"
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 2)
    p = prompts_of(name, [40], seed=3)[0]
    seen, used = [], {}

    def hook(step_no, layer_no, op, tensor):
        if op == "hidden_post_ffn":
            seen.append(f64(tensor))
        if op == "experts":
            used[layer_no] = tensor.cpu().numpy().copy()
    model.op_hook = hook
    slot = cache.open_sequence()
    step(model, cache, [StepEntry(slot, p, [])])
    model.op_hook = None
    cache.close_sequence(slot)
    want = []
    plain.forward(CONFIGS[name][0], weights_of(folders, name), p, experts_of=used, layers_out=want)
    assert len(seen) == len(want) == len(CONFIG_R["layers"])
    for i, (g, w) in enumerate(zip(seen, want)):
        close(g, w, dtype, f"the sum of the copies after layer {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R", "S"])
def test_portions_down_to_two_tokens_and_token_by_token_from_the_start(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    p = prompts_of(name, [150], seed=5)[0]
    want = want_logits(folders, name, p)
    rows = {}
    for portions in ([150], [1], [2], [3, 2, 1, 16, 15, 17, 64], [63, 1, 1, 64, 2], [100, 1], [69, 1, 1, 1, 78]):
        rows[tuple(portions)], used = run_cut(model, cache, p, portions)
        model_close(folders, name, dtype, p, rows[tuple(portions)], used, f"{name} {dtype} portions {portions}")
    if dtype == "float32":
        # sums walk keys and channels in one order whatever the cut: the float32 answers agree to the last bits
        for portions, got in rows.items():
            np.testing.assert_allclose(got, rows[(150,)], rtol=0, atol=2e-5 * np.abs(want).max(), err_msg=str(portions))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R", "S", "U"])
def test_long_decoding_across_page_borders_and_stretches(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    p = prompts_of(name, [5 + 280], seed=6)[0]
    got, used = run_cut(model, cache, p, [5, 1])
    model_close(folders, name, dtype, p, got, used, f"{name} {dtype} 280 tokens decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R", "S"])
def test_unequal_batches_against_each_alone_with_slots_and_pages_used_again(folders, name, dtype):
    """Three batches through a cache too small for two of them: the slots and pages
    of finished requests, with their old rows, go to new ones.  In a batch every
    request is decoded to its own length and leaves when it ends."""
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 7, max_slots=4)
    batches = [[(5, 9), (70, 3), (17, 20), (1, 12)], [(64, 1), (130, 6), (3, 33)], [(40, 8), (128, 2), (9, 9), (2, 2)]]
    for bi, batch in enumerate(batches):
        prompts = prompts_of(name, [a + b for a, b in batch], seed=20 + bi)
        slots = [cache.open_sequence() for _ in batch]
        got, used = [[] for _ in batch], [[] for _ in batch]
        listen = Choices(model)
        entries = [StepEntry(slots[i], p[:plen], list(range(plen))) for i, ((plen, _), p) in enumerate(zip(batch, prompts))]
        flat = step(model, cache, entries).float().cpu().numpy()
        o = 0
        for i, (e, rows) in enumerate(zip(entries, listen.take([len(e.tokens) for e in entries]))):
            got[i].append(flat[o:o + len(e.want)])
            used[i].append(rows)
            o += len(e.want)
        live, t = list(range(len(batch))), 0
        while True:
            live = [i for i in live if t < batch[i][1]]
            if not live:
                break
            flat = step(model, cache, [StepEntry(slots[i], [prompts[i][batch[i][0] + t]], [0]) for i in live]).float().cpu().numpy()
            for (j, i), rows in zip(enumerate(live), listen.take([1] * len(live))):
                got[i].append(flat[j:j + 1])
                used[i].append(rows)
                if t + 1 >= batch[i][1]:
                    cache.close_sequence(slots[i])
            t += 1
        listen.close()
        for i in range(len(batch)):
            model_close(folders, name, dtype, prompts[i], np.concatenate(got[i]), join(used[i]), f"{name} {dtype} batch {bi} request {i}")
        assert cache.open_slots() == []
    assert all(free == 7 for free in cache.free_pages())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["R", "S"])
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
        # bfloat16: a token routed to another expert than in the plain implementation may pick another token
        assert all(ok) if dtype == "float32" else sum(ok) >= 0.8 * len(ok), (use_graph, ok)
    if dtype == "float32":
        assert results[1].tokens == plain.greedy(cfg, w, prompts[1], 6)


def test_trace_replay_and_command_line(folders, tmp_path):
    """bin/trace_run with a batch that starts together and shrinks, and llmgen with token ids."""
    name = "R"
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
