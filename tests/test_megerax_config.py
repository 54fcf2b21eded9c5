"""The Megerax design without a device: its configuration and its errors, the
plan's parts, tensor names, schedule and cache requests, and the plain
implementation against closed forms."""
import copy
import math

import numpy as np
import pytest

import go_tinygrad_b200 as lib
import plain_megerax as plain
from go_tinygrad_b200.cache import KVRequest, StateRequest
from go_tinygrad_b200.config.megerax import MegeraxConfig
from go_tinygrad_b200.config.registry import find_architecture
from go_tinygrad_b200.parts import build_part
from go_tinygrad_b200.parts.plan import plan_weight_specs
from go_tinygrad_b200.parts.position import rotary_frequencies

SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}


def attention(heads, kv_heads, dim, vdim, scale, conv=None, window=None, rot=None, softcap=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    for key, value in (("conv", conv), ("rot", rot), ("softcap", softcap), ("kv_from", kv_from)):
        if value is not None:
            m[key] = value
    if window is not None:
        m["mask"] = {"size": window}
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot, window=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def delta(heads, kv_heads, dim, vdim, conv=None, decay_rank=None, gate_rank=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim}
    for key, value in (("conv", conv), ("decay_rank", decay_rank), ("gate_rank", gate_rank)):
        if value is not None:
            m[key] = value
    return m


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


SMALL = {
    "architecture": "Megerax", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "layers": [
        layer("attention", attention(4, 2, 12, 6, 0.3, conv=4, window=9, rot={"dims": 8, "base": 100.0, "scaling": SCALING}, softcap=7.0), 24),
        layer("channel_delta", delta(4, 2, 10, 6, conv=2)),
        layer("latent_attention", latent(3, 8, 4, 6, 12, 10, 0.25, {"dims": 4, "base": 50.0}), 16),
        layer("attention", attention(4, 2, 12, 6, 0.2, conv=2, rot={"dims": 8, "base": 100.0, "scaling": SCALING}, kv_from=0)),
    ],
}


def test_configuration_reads_every_key_and_writes_it_back():
    cfg = MegeraxConfig.from_json(SMALL)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_scale) == (97, 40, 1e-5, 0.5)
    a, d, l, b = (x.mixer for x in cfg.layers)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.window, a.softcap, a.kv_from) == (4, 2, 12, 6, 4, 9, 7.0, None)
    assert (a.rot.dims, a.rot.base, a.rot.scaling.factor, a.rot.scaling.original) == (8, 100.0, 8.0, 64.0)
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv, d.decay_rank) == (4, 2, 10, 6, 2, None)
    assert (l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.q_rank, l.window) == (3, 8, 4, 6, 12, 10, None)
    assert (b.kv_from, b.window, b.softcap, b.conv) == (0, None, None, 2)
    assert cfg.layers[1].mlp is None and cfg.layers[0].mlp.ff == 24
    again = MegeraxConfig.from_json(cfg.to_json())
    assert again == cfg
    assert find_architecture(SMALL).read_config(SMALL) == cfg
    plain_scale = dict(SMALL)
    del plain_scale["logit_scale"]
    assert MegeraxConfig.from_json(plain_scale).logit_scale == 1.0


@pytest.mark.parametrize("path,value,needle", [
    (("layers", 0, "type"), "attention_9", "type"),
    (("layers", 0, "mixer", "heads"), 3, "cannot share"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 14, "at most"),
    (("layers", 0, "mixer", "rot", "scaling", "high"), 0.5, "high"),
    (("layers", 0, "mixer", "scale"), None, "scale"),
    (("layers", 1, "mixer", "kv_heads"), 3, "cannot share"),
    (("layers", 2, "mixer", "rot_dim"), 5, "even"),
    (("layers", 2, "mixer", "rot"), None, "rot"),
    (("layers", 2, "mixer", "q_rank"), None, "q_rank"),
    (("layers", 3, "mixer", "kv_from"), 3, "earlier"),
    (("layers", 3, "mixer", "kv_from"), 1, "no keys and values"),
    (("layers", 3, "mixer", "dim"), 16, "must equal"),
    (("layers", 1, "mlp"), {"kind": "moe"}, "kind"),
    (("norm",), None, "eps"),
    (("layers",), [], "non-empty"),
])
def test_configuration_errors_name_the_key(path, value, needle):
    raw = copy.deepcopy(SMALL)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(lib.ConfigError) as e:
        MegeraxConfig.from_json(raw)
    assert needle in str(e.value)


def test_plan_parts_tensors_schedule_and_cache_requests():
    arch = find_architecture(SMALL)
    plan = arch.plan(arch.read_config(SMALL))
    assert [e.cache for e in plan.schedule] == [None, None, None, 0]
    names = {s.name: s for s in plan_weight_specs(plan)}
    for name, shape in {"embed": (97, 40), "embed.norm": (40,), "head": (97, 40), "final.norm": (40,),
                        "l0.mix.q": (48, 40), "l0.mix.q.b": (48,), "l0.mix.k": (24, 40), "l0.mix.v": (12, 40), "l0.mix.v.b": (12,),
                        "l0.mix.q.conv": (48, 4), "l0.mix.v.conv": (12, 4), "l0.mix.q.norm": (12,), "l0.mix.k.norm": (12,),
                        "l0.mix.g": (24, 40), "l0.mix.o": (40, 24), "l0.mlp.gate": (24, 40), "l0.mlp.down": (40, 24),
                        "l1.mix.q": (20, 40), "l1.mix.v": (24, 40), "l1.mix.b": (4, 40), "l1.mix.A_log": (4,), "l1.mix.dt_bias": (40,),
                        "l1.mix.a1": (-1, 40), "l1.mix.a2": (40, -1), "l1.mix.g2": (24, -1), "l1.mix.norm": (6,), "l1.mix.k.conv": (20, 2),
                        "l2.mix.dq": (10, 40), "l2.mix.dq.norm": (10,), "l2.mix.uq": (36, 10), "l2.mix.dkv": (16, 40),
                        "l2.mix.dkv.norm": (12,), "l2.mix.uk": (24, 12), "l2.mix.uv": (18, 12), "l2.mix.sink": (3,), "l2.mix.o": (40, 18),
                        "l3.mix.q": (48, 40), "l3.mix.q.conv": (48, 2), "l3.mix.q.norm": (12,), "l3.mix.g": (24, 40)}.items():
        assert names[name].shape == shape, name
    for absent in ("l1.norm2", "l3.mix.k", "l3.mix.v", "l3.mix.k.b", "l3.mix.k.conv", "l3.mix.k.norm", "l3.norm2", "l1.mlp.gate"):
        assert absent not in names
    blocks = [build_part("block", spec.block) for spec in plan.layers]
    # layer 3 reads layer 0's keys through no window at all: the cache keeps every key, whatever layer 0's own window
    assert blocks[0].cache_requests() == [KVRequest(2, 12, None, value_dim=6), StateRequest("conv", (3, 48 + 24 + 12), "float32")]
    windowed = copy.deepcopy(SMALL)
    for i, size in ((0, 9), (3, 30)):
        windowed["layers"][i]["mixer"]["mask"] = {"size": size}
    kept = build_part("block", arch.plan(arch.read_config(windowed)).layers[0].block).cache_requests()[0]
    assert kept == KVRequest(2, 12, 30, value_dim=6)
    assert blocks[1].cache_requests() == [StateRequest("delta", (4, 10, 6), "float32"), StateRequest("conv", (1, 20 + 20 + 24), "float32")]
    assert blocks[2].cache_requests() == [KVRequest(1, 16, None, planes=1)]
    assert blocks[3].cache_requests() == [StateRequest("conv", (1, 48), "float32")]      # queries only: the keys are layer 0's
    # a rank the configuration names is the tensor's size; one it does not name is the checkpoint's
    raw = copy.deepcopy(SMALL)
    raw["layers"][1]["mixer"].update({"decay_rank": 5, "gate_rank": 3})
    names = {s.name: s for s in plan_weight_specs(arch.plan(arch.read_config(raw)))}
    assert names["l1.mix.a1"].shape == (5, 40) and names["l1.mix.g2"].shape == (24, 3)


def test_scaled_frequencies_of_package_and_plain_implementation():
    for dims, base in ((8, 100.0), (64, 10000.0), (32, 500000.0)):
        ours = rotary_frequencies(dims, base, {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                               "original_max_position_embeddings": 64})
        np.testing.assert_allclose(ours, plain.frequencies(dims, base, SCALING), rtol=1e-14)
        np.testing.assert_allclose(rotary_frequencies(dims, base), plain.frequencies(dims, base), rtol=1e-14)
    f = plain.frequencies(8, 100.0, SCALING)
    raw = [100.0 ** (-2 * i / 8) for i in range(4)]
    # wavelengths 6.3, 19.9, 62.8, 198.7 against 64/4 = 16 and 64/1 = 64: kept, blended, blended, divided
    assert f[0] == raw[0] and f[3] == raw[3] / 8.0 and raw[1] / 8.0 < f[1] < raw[1] and raw[2] / 8.0 < f[2] < raw[2]


def test_plain_implementation_against_closed_forms():
    rng = np.random.default_rng(0)
    # a convolution whose taps are (0, .., 0, 1) changes nothing; (1, 0) delays by one token
    u = rng.standard_normal((7, 3))
    np.testing.assert_allclose(plain.causal_conv(u, np.array([[0, 0, 1.0]] * 3)), u)
    np.testing.assert_allclose(plain.causal_conv(u, np.array([[1.0, 0]] * 3)), np.concatenate([np.zeros((1, 3)), u[:-1]]))
    # rotation keeps lengths, pairs as named, and a rotated dot product depends on the distance only
    x = rng.standard_normal((5, 2, 8))
    f = plain.frequencies(4, 10.0)
    for pairing in ("interleaved", "half"):
        r = plain.rotate(x, np.arange(5), f, pairing)
        np.testing.assert_allclose(np.linalg.norm(r, axis=-1), np.linalg.norm(x, axis=-1))
        np.testing.assert_allclose(r[..., 4:], x[..., 4:])
        np.testing.assert_allclose(r[0], x[0])
    q, k = rng.standard_normal((1, 1, 4)), rng.standard_normal((1, 1, 4))
    dots = [float((plain.rotate(q, [p + 3], f, "half") * plain.rotate(k, [p], f, "half")).sum()) for p in (0, 5, 40)]
    np.testing.assert_allclose(dots, dots[0])
    one = plain.rotate(np.array([[[1.0, 0, 0, 0]]]), [1], f, "interleaved")[0, 0]
    np.testing.assert_allclose(one, [math.cos(1.0), math.sin(1.0), 0, 0], atol=1e-15)
    one = plain.rotate(np.array([[[1.0, 0, 0, 0]]]), [1], f, "half")[0, 0]
    np.testing.assert_allclose(one, [math.cos(1.0), 0, math.sin(1.0), 0], atol=1e-15)
    # attention: a window of one returns the token's own value; a cap bounds what a score can do; a sink of
    # +infinity's worth leaves nothing, one of -infinity's worth changes nothing
    q, k, v = rng.standard_normal((6, 2, 4)), rng.standard_normal((6, 1, 4)), rng.standard_normal((6, 1, 3))
    np.testing.assert_allclose(plain.attend(q, k, v, 1.0, window=1), np.broadcast_to(v, (6, 2, 3)))
    big = plain.attend(1000 * q, k, v, 1.0, softcap=1e-9)
    np.testing.assert_allclose(big[3, 0], v[:4, 0].mean(axis=0), atol=1e-6)
    np.testing.assert_allclose(plain.attend(q, k, v, 1.0, sinks=np.array([-800.0, -800.0])), plain.attend(q, k, v, 1.0))
    assert np.abs(plain.attend(q, k, v, 1.0, sinks=np.array([60.0, 60.0]))).max() < 1e-15
    one_key = plain.attend(q[:1], k[:1], v[:1], 1.0, sinks=np.array([0.0, 0.0]))
    s = (q[0] @ k[0, 0])
    np.testing.assert_allclose(one_key[0], (np.exp(s) / (np.exp(s) + 1.0))[:, None] * v[0])
    # the delta rule: with beta = 1 and no decay the state returns v for its own unit key, and a second write
    # along the same key replaces the first
    kk = np.zeros((2, 4)); kk[:, 1] = 1.0
    vv = rng.standard_normal((2, 3))
    out = plain.delta_rule(kk, kk, vv, np.ones(2), np.ones((2, 4)))
    np.testing.assert_allclose(out, vv)
    # a decay of one half on every row halves what an orthogonal, earlier write returns
    k2 = np.eye(4)[:2]
    out = plain.delta_rule(np.stack([k2[0], k2[0]]), k2, vv, np.ones(2), np.full((2, 4), 0.5))
    np.testing.assert_allclose(out[1], 0.5 * vv[0])
    assert abs(plain.gelu_tanh(1.0) - 0.8411919906082768) < 1e-12 and plain.gelu_tanh(0.0) == 0.0
