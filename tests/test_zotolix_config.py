"""The Zotolix design without a device: its configuration and errors, the plan's
tensor names and cache requests, the cache's handling of keys seen within
stretches of positions, and the plain implementation against closed forms."""
import copy

import numpy as np
import pytest
import torch

import go_tinygrad_b200 as lib
import plain_zotolix as plain
from go_tinygrad_b200.cache import Cache, KVRequest
from go_tinygrad_b200.config import ConfigError, ZotolixConfig
from go_tinygrad_b200.config.registry import find_architecture
from go_tinygrad_b200.parts import build_part, plan_weight_specs


def mixer(heads, kv_heads, dim, vdim, chunk, scale, dims, base, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix,
         "rot": {"dims": dims, "base": base}}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return m


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


CONFIG = {
    "architecture": "Zotolix", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
    "residual_mult": 0.75, "streams": 3,
    "layers": [
        {"type": "attention", "mixer": mixer(3, 3, 8, 6, 5, 0.3, 4, 100.0), "mlp": moe(20, 5, 2)},
        {"type": "attention_2", "mixer": mixer(4, 2, 4, 12, 9, 0.2, 4, 50.0, v_mix=True), "mlp": None},
        {"type": "attention", "mixer": mixer(2, 2, 16, 12, None, 0.5, 2, 7.0, v_mix=True), "mlp": moe(12, 2, 1)},
    ],
}


def test_configuration_reads_every_size_and_constant():
    cfg = ZotolixConfig.from_json(CONFIG)
    assert (cfg.vocab, cfg.width, cfg.streams, cfg.residual_mult, cfg.embedding_scale, cfg.norm_eps) == (97, 48, 3, 0.75, 2.5, 1e-5)
    m = cfg.layers[1].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.chunk, m.scale, m.rot.dims, m.rot.base, m.v_mix) == (4, 2, 4, 12, 9, 0.2, 4, 50.0, True)
    assert cfg.layers[2].mixer.chunk is None and cfg.layers[1].mlp is None and cfg.layers[0].mlp.top == 2
    assert ZotolixConfig.from_json(cfg.to_json()) == cfg
    assert find_architecture(CONFIG).read_config(CONFIG) == cfg
    plainer = {k: v for k, v in CONFIG.items() if k not in ("streams", "residual_mult", "embedding")}
    cfg = ZotolixConfig.from_json(plainer)
    assert (cfg.streams, cfg.residual_mult, cfg.embedding_scale) == (None, 1.0, 1.0)


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "attention_3", "type"), (("layers", 1, "mixer", "heads"), 3, "share"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 3, "rot.dims"),
    (("layers", 2, "mixer", "vdim"), 6, "blends"), (("layers", 2, "mixer", "kv_heads"), 1, "blends"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"), (("layers", 0, "mlp", "router", "top"), 6, "experts"),
    (("layers", 0, "mlp", "kind"), "dense", "ff"), (("streams",), 9, "streams"), (("norm",), None, "eps"),
    (("layers", 1, "mixer", "v_mix"), 1, "v_mix"), (("layers",), [], "layers"), (("width",), -4, "width"),
])
def test_configuration_errors_name_the_key(path, value, word):
    raw = copy.deepcopy(CONFIG)
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        ZotolixConfig.from_json(raw)


def test_plan_names_tensors_and_asks_the_cache_for_what_the_layers_keep():
    arch = find_architecture(CONFIG)
    plan = arch.plan(arch.read_config(CONFIG))
    names = {s.name: s for s in plan_weight_specs(plan)}
    for n, shape in {"embed": (97, 48), "l0.mix.q": (24, 48), "l0.mix.q.b": (24,), "l0.mix.k.b": (24,), "l0.mix.v": (18, 48),
                     "l0.mix.o": (48, 18), "l1.mix.g": (4, 48), "l1.mix.v.b": (24,), "l1.mix.o": (48, 48), "l2.mix.vmix": (),
                     "l0.hc1.in": (3,), "l0.hc2.mix": (3, 3), "l1.hc1.out": (3,), "l0.mlp.router": (5, 48),
                     "l0.mlp.e4.up": (20, 48), "l2.mlp.e1.down": (48, 12), "final.norm": (48,)}.items():
        assert tuple(names[n].shape) == shape, n
    assert "l0.mix.g" not in names and "l1.hc2.in" not in names and "l0.mix.vmix" not in names and "head" not in names
    assert "l0.mlp.e0.gate" not in names
    assert names["l1.mix.vmix"].optional and not names["l2.mix.vmix"].optional      # the first blending layer's is never read
    blocks = [build_part("block", layer.block) for layer in plan.layers]
    assert blocks[0].cache_requests() == [KVRequest(3, 8, None, value_dim=6, chunk=5)]
    assert blocks[1].cache_requests() == [KVRequest(2, 4, None, value_dim=12, chunk=9)]
    assert blocks[2].cache_requests() == [KVRequest(2, 16, None, value_dim=12, chunk=None)]
    # without `streams`: one copy, no tensors of the block's own
    plainer = {k: v for k, v in CONFIG.items() if k != "streams"}
    names = {s.name for s in plan_weight_specs(arch.plan(arch.read_config(plainer)))}
    assert not any(".hc" in n for n in names)


def test_cache_keeps_values_of_their_own_width_and_gives_back_pages_before_the_stretch():
    reqs = [[KVRequest(2, 16, None, value_dim=24, chunk=100)], [KVRequest(2, 16, None, value_dim=24, chunk=100)],
            [KVRequest(1, 8, None, chunk=64)]]
    cache = Cache(reqs, [None, None, None], max_tokens=64 * 8, max_slots=2, dtype=torch.float32, device="cpu")
    kv = cache.handles[1].kv
    assert (kv.head_dim, kv.value_dim, kv.chunk) == (16, 24, 100)
    assert tuple(kv.k.shape[1:]) == (2, 64, 16) and tuple(kv.v.shape[1:]) == (2, 64, 24)
    assert kv.k.stride(0) == kv.v.stride(0) == 2 * 64 * (16 + 24) == kv.page_stride
    kv.k[3, 1, 63, 15] = 5.0
    kv.v[3, 0, 0, 0] = 7.0                                     # the value block starts where the key block ends
    flat = cache.groups[0].storage[1, 3]
    assert flat[2 * 64 * 16 - 1] == 5.0 and flat[2 * 64 * 16] == 7.0
    slot = cache.open_sequence()
    cache.reserve(slot, 330)
    cache.advance(slot, 199)          # the next token, 199, still sees 100..199: page 0 (0..63) is gone, page 1 holds 100
    assert cache.free_pages() == [8 - 6 + 1, 8 - 6 + 3]       # stretches of 64: the token at 199 sees 192..199 only
    cache.advance(slot, 1)            # the next token, 200, opens a stretch: pages 0..2 (up to 191) are gone
    assert cache.groups[0].pages_of[slot][:4] == [-1, -1, -1, cache.groups[0].pages_of[slot][3]]
    with pytest.raises(lib.cache.CacheMisuse):
        cache.truncate(slot, 150)
    cache.truncate(slot, 200)
    cache.close_sequence(slot)
    assert cache.free_pages() == [8, 8]


def test_plain_implementation_against_closed_forms():
    rng = np.random.default_rng(0)
    # a rotation keeps lengths, leaves the channels from `dims` on alone, and position 0 alone
    x = rng.standard_normal((5, 2, 10))
    r = plain.rotate_heads(x, np.arange(5), 6, 100.0)
    np.testing.assert_allclose(np.linalg.norm(r, axis=-1), np.linalg.norm(x, axis=-1))
    np.testing.assert_array_equal(r[..., 6:], x[..., 6:])
    np.testing.assert_allclose(r[0], x[0])
    a = 3 * 100.0 ** (-2.0 / 6)                                # position 3, pair 1: channels 1 and 4
    np.testing.assert_allclose(r[3, 0, 1], x[3, 0, 1] * np.cos(a) - x[3, 0, 4] * np.sin(a))
    np.testing.assert_allclose(r[3, 0, 4], x[3, 0, 4] * np.cos(a) + x[3, 0, 1] * np.sin(a))
    # stretches of 4: position 5 sees 4 and 5, position 4 itself alone, position 3 sees 0..3
    assert [j for j in range(8) if plain.chunk_visible(5, j, 4)] == [4, 5]
    assert [j for j in range(8) if plain.chunk_visible(4, j, 4)] == [4]
    assert [j for j in range(8) if plain.chunk_visible(3, j, 4)] == [0, 1, 2, 3]
    assert [j for j in range(8) if plain.chunk_visible(5, j, None)] == [0, 1, 2, 3, 4, 5]
    q, k, v = rng.standard_normal((8, 2, 3)), rng.standard_normal((8, 1, 3)), rng.standard_normal((8, 1, 2))
    out = plain.attend(q, k, v, 0.5, 4)
    np.testing.assert_allclose(out[4, 1], v[4, 0])             # the first token of a stretch sees itself only
    s = np.array([q[6, 0] @ k[j, 0] for j in (4, 5, 6)]) * 0.5
    p = np.exp(s) / np.exp(s).sum()
    np.testing.assert_allclose(out[6, 0], p @ v[4:7, 0])
    # experts: a score of s on the input of a squared relu is s^2 on its output
    h = rng.standard_normal((6, 5))
    router, ups, downs = rng.standard_normal((3, 5)), rng.standard_normal((3, 4, 5)), rng.standard_normal((3, 5, 4))
    idx, score = plain.choose_experts(h, router, 2)
    assert (np.diff(score, axis=-1) <= 0).all() and (score > 0).all() and (score < 1).all()
    got = plain.mixture(h, router, ups, downs, 2)
    want = np.zeros_like(got)
    for t in range(6):
        for e, s_ in zip(idx[t], score[t]):
            want[t] += s_ ** 2 * plain.expert(h[t], ups[e], downs[e])
    np.testing.assert_allclose(got, want)
    # copies: in = 1/S, mix = identity, out = 1 is the ordinary residual sum on every copy
    xs = np.stack([rng.standard_normal((4, 5))] * 3)
    y = rng.standard_normal((4, 5))
    np.testing.assert_allclose(plain.streams_read(xs, [1 / 3] * 3), xs[0])
    np.testing.assert_allclose(plain.streams_write(xs, y, np.eye(3), np.ones(3), 0.5), xs + 0.5 * y)
    mix = rng.standard_normal((3, 3))
    new = plain.streams_write(xs * np.arange(1, 4)[:, None, None], y, mix, [1, 2, 3], 2.0)
    np.testing.assert_allclose(new[2], (mix[0, 2] + 2 * mix[1, 2] + 3 * mix[2, 2]) * xs[0] + 6 * y)   # mix is [from, to]
