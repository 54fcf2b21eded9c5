"""The Megerax decoder as a plan of parts.

The embedded tokens pass an RMS norm (``token_embedding`` with ``norm``); every
layer is a ``pre_norm`` block around one of three mixers and, where the layer
has one, a gated feed-forward whose gate passes the tanh form of gelu
(``swiglu`` with ``activation``); a final RMS norm, an untied head and a
multiplier on the logits (``lm_head`` with ``scale``) close the model.  The
mixers: ``gqa_attention`` with biased projections, a causal convolution over q,
k and v, weighted norms per query and key head, a rotation of interleaved pairs
under wavelength scaling, capped scores, a sliding window and a sigmoid gate on
all channels (a layer with ``kv_from`` reads the cache of the layer it names:
the schedule entry's ``cache``); ``latent_attention`` with queries through a
latent of their own, half-split pairs and a sink per head; and ``gated_delta``,
the delta rule with a decay per head and key channel.  Tensor names: ``embed``,
``embed.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``final.norm``, ``head``.  The reference has no such architecture.
"""
from __future__ import annotations

from ..config.megerax import MegeraxConfig
from ..config.registry import Architecture, register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


def _norm(cfg: MegeraxConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name})


def _rotary(rot, head_dim: int, pairing: str) -> PartSpec:
    if rot is None:
        return PartSpec("none", {})
    scaling = None
    if rot.scaling is not None:
        s = rot.scaling
        scaling = {"factor": s.factor, "low_freq_factor": s.low, "high_freq_factor": s.high,
                   "original_max_position_embeddings": s.original}
    return PartSpec("rotary", {"head_dim": head_dim, "rotary_dim": rot.dims, "theta": rot.base, "pairing": pairing,
                               "scaling": scaling})


def _kept_window(cfg: MegeraxConfig, i: int):
    """How many keys layer i's cache keeps: what the longest-sighted of the layers that read it sees
    (itself and those whose ``kv_from`` names it); None, all keys, if one of them has no window."""
    windows = [cfg.layers[i].mixer.window] + [layer.mixer.window for layer in cfg.layers
                                              if layer.type == "attention" and layer.mixer.kv_from == i]
    return None if any(w is None for w in windows) else max(windows)


def _attention(cfg: MegeraxConfig, i: int) -> PartSpec:
    m, p = cfg.layers[i].mixer, f"l{i}.mix."
    own = m.kv_from is None
    params = {"hidden_size": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
              "scale": m.scale, "window": m.window, "softcap": m.softcap, "own_kv": own,
              "position": _rotary(m.rot, m.dim, "interleaved"),
              "q": p + "q", "o": p + "o", "q_bias": p + "q.b", "output_gate": p + "g",
              "qk_norm": "weight", "q_norm": p + "q.norm", "norm_eps": cfg.norm_eps}
    conv = {"taps": m.conv, "q": p + "q.conv"} if m.conv else None
    if own:
        params["cache_window"] = _kept_window(cfg, i)
        params.update({"k": p + "k", "v": p + "v", "k_bias": p + "k.b", "v_bias": p + "v.b", "k_norm": p + "k.norm"})
        if conv:
            conv.update({"k": p + "k.conv", "v": p + "v.conv"})
    params["conv"] = conv
    return PartSpec("gqa_attention", params)


def _latent(cfg: MegeraxConfig, i: int) -> PartSpec:
    m, p = cfg.layers[i].mixer, f"l{i}.mix."
    return PartSpec("latent_attention", {
        "hidden_size": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
        "kv_rank": m.kv_rank, "window": m.window, "scale": m.scale, "eps": cfg.norm_eps,
        "position": _rotary(m.rot, m.rot_dim, "half"),
        "q": p + "uq", "q_latent": {"rank": m.q_rank, "down": p + "dq", "norm": p + "dq.norm"},
        "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv", "sinks": p + "sink", "o": p + "o"})


def _delta(cfg: MegeraxConfig, i: int) -> PartSpec:
    m, p = cfg.layers[i].mixer, f"l{i}.mix."
    return PartSpec("gated_delta", {
        "hidden_size": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
        "conv_taps": m.conv, "eps": cfg.norm_eps, "unit_eps": 1e-6, "decay_rank": m.decay_rank, "gate_rank": m.gate_rank,
        "q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv",
        "beta": p + "b", "a_log": p + "A_log", "decay_down": p + "a1", "decay_up": p + "a2", "dt_bias": p + "dt_bias",
        "gate_down": p + "g1", "gate_up": p + "g2", "norm": p + "norm", "o": p + "o"})


_MIXERS = {"attention": _attention, "latent_attention": _latent, "channel_delta": _delta}


def megerax_plan(cfg: MegeraxConfig) -> ModelPlan:
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1"), "mixer": _MIXERS[layer.type](cfg, i),
                 "feed_forward_norm": None, "feed_forward": None}
        if layer.mlp is not None:
            parts["feed_forward_norm"] = _norm(cfg, p + "norm2")
            parts["feed_forward"] = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff,
                                                        "activation": "gelu_tanh", "gate": p + "mlp.gate",
                                                        "up": p + "mlp.up", "down": p + "mlp.down"})
        layers.append(LayerSpec(PartSpec("pre_norm", parts)))
        schedule.append(ScheduleEntry(layer=i, cache=getattr(layer.mixer, "kv_from", None)))
    plan = ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed",
                                               "norm": {"weight": "embed.norm", "eps": cfg.norm_eps}}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "head",
                                  "scale": cfg.logit_scale}),
        stop_tokens=(),
        max_position=None,
    )
    plan.check()
    return plan


MEGERAX = register_architecture(Architecture(
    names=("Megerax", "megerax"),
    read_config=MegeraxConfig.from_json,
    plan=megerax_plan,
))
