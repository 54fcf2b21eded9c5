"""The Zotolix decoder as a plan of parts.

Every layer is a ``hyper_connections`` block (the hidden state in `streams`
copies; a sublayer reads a weighted sum of them through an RMS norm and writes
back into all of them, times ``residual_mult``) around grouped-query attention
(``gqa_attention`` with biased projections, a rotation of a head's first
channels, keys seen within stretches of ``mask.size`` positions, values of a
size of their own that are blended with the first blending layer's, and either
unit-norm queries and keys or a sigmoid gate per head) and a mixture of
squared-relu experts whose sigmoid router score scales the expert's input
(``routed_experts``).  The embedded tokens are multiplied by
``embedding.scale``; a final RMS norm over the sum of the copies and the
embedding table as the head close the model.  Tensor names: ``embed``,
``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.mix.q|k|v[.b]|vmix|g|o``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.up|down``,
``final.norm``.  The reference has no such architecture.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.zotolix import ZotolixConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, default_schedule


def _norm(cfg: ZotolixConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name})


def _mixer(cfg: ZotolixConfig, i: int, first_blend: int) -> PartSpec:
    layer = cfg.layers[i]
    m, p = layer.mixer, f"l{i}.mix."
    if m.rot is not None:
        position = PartSpec("rotary", {"head_dim": m.dim, "rotary_dim": m.rot.dims, "theta": m.rot.base, "pairing": "half"})
    else:
        position = PartSpec("none", {})
    blend = None
    if m.v_mix:
        blend = {"role": "source" if i == first_blend else "blend", "weight": p + "vmix", "key": "values_of_first_blend"}
    return PartSpec("gqa_attention", {
        "hidden_size": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
        "scale": m.scale, "chunk": m.chunk, "position": position,
        "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o",
        "q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b",
        "qk_norm": "unit" if layer.type == "attention" else None, "norm_eps": cfg.norm_eps,
        "head_gate": p + "g" if layer.type == "attention_2" else None,
        "value_blend": blend})


def _feed_forward(cfg: ZotolixConfig, i: int) -> PartSpec:
    mlp, p = cfg.layers[i].mlp, f"l{i}.mlp."
    return PartSpec("routed_experts", {"hidden_size": cfg.width, "intermediate_size": mlp.ff,
                                       "n_experts": mlp.experts, "top": mlp.top, "router": p + "router",
                                       "gate": None, "up": p + "e{e}.up", "down": p + "e{e}.down",
                                       "activation": "relu2", "scoring": "sigmoid", "weight_on": "input"})


def zotolix_plan(cfg: ZotolixConfig) -> ModelPlan:
    blending = [i for i, layer in enumerate(cfg.layers) if layer.mixer.v_mix]
    first_blend = blending[0] if blending else -1
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, i, first_blend),
                 "feed_forward_norm": None, "feed_forward": None,
                 "hidden_size": cfg.width, "copies": cfg.streams, "update_scale": cfg.residual_mult,
                 "mixer_links": p + "hc1", "feed_forward_links": p + "hc2"}
        if layer.mlp is not None:
            parts["feed_forward_norm"] = _norm(cfg, p + "norm2")
            parts["feed_forward"] = _feed_forward(cfg, i)
        layers.append(LayerSpec(PartSpec("hyper_connections", parts)))
    plan = ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed",
                                               "scale": cfg.embedding_scale}),
        layers=tuple(layers),
        schedule=default_schedule(len(layers)),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed", "tied": True}),
        stop_tokens=(),
        max_position=None,
    )
    plan.check()
    return plan


ZOTOLIX = register_architecture(Architecture(
    names=("Zotolix", "zotolix"),
    read_config=ZotolixConfig.from_json,
    plan=zotolix_plan,
))
