"""Arrangements of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(model/llama.go:1087-1097, 1311-1314, 1425).  Its parameters are the four
nested specs ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and
``feed_forward``; the last two may be None for a layer that has a mixer only.
The additions are not done here: each update is left
pending on the residual stream and the next norm (of this layer, of the next
one, or the final one) adds it in float32 while it normalises -- unless the
part, offered the stream (`emit_update`), has added its update in its last
product's epilogue already and returns None.

``output_norm``: x += norm1(mixer(x)); x += norm2(feed_forward(x)): the norm
stands on a sublayer's output and the sublayers read the hidden state itself
(rounded to the compute dtype for their products).  Same four nested specs as
``pre_norm``; the feed-forward and its norm may be None.  The norms must be of
kind ``rmsnorm`` (the one norm whose fused form with the addition exists).  A
sublayer's update may be float32 or of the compute dtype; norm and addition are
float32, and the kernel that adds also leaves the rounded hidden state for the
next sublayer (`ResidualStream.image`); a part may leave the bias of its last
projection for that kernel to add (`StepContext.update_bias`).  Nothing is left pending.  The reference
has no such arrangement.

``hyper_connections``: the hidden state in S copies x_1..x_S (all equal to the
embedding output at the start).  Sublayer q (the mixer, then the feed-forward)
reads u = sum_s in_q[s] x_s through its norm, and its output y goes back as
x_t <- sum_s mix_q[s, t] x_s + m out_q[t] y, all copies at once from the old
ones; at the end the hidden state is the sum of the copies.  Same four nested
specs as ``pre_norm`` (the feed-forward and its norm may be None; the norms of
kind ``rmsnorm``) and ``hidden_size``, ``copies`` (S, or None: one copy with
in = mix = out = 1, which is the ordinary residual sum x += m y, and no tensors
of its own), ``update_scale`` (m), ``mixer_links`` and ``feed_forward_links``
(prefixes of the tensors ``.in`` [S], ``.out`` [S], ``.mix`` [S, S], indexed
[from, to]).  Nothing is added here: a sublayer's output is left pending on
the stream with its links, and the kernel that reads the copies for the next
sublayer (of this layer, the next one, or the final norm) applies it on the
way, in float32.  The reference has no such arrangement.

``concat_projection``: x <- W [x | kept], a projection of the hidden state side
by side with a tensor an earlier part has kept for the step under the name
``source`` in the step's shared values (the token embedding keeps its output
as "embedding_output" when asked to).  It replaces the hidden state instead
of adding to it, holds no cache, and can stand anywhere in the schedule, as
often as wanted.  Parameters: ``hidden_size``, ``weight`` (tensor name,
[hidden, 2 hidden], the hidden state's columns first), ``source``.  The
reference has no such part.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..cache import CacheHandle
from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Block, ResidualStream, Runtime, StepContext, register_part


def _hidden(stream: ResidualStream):
    """The hidden state as a value: the residual with its pending update added."""
    if stream.pending is None:
        return stream.residual.clone()
    return stream.residual + stream.pending.float()


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    sub_parts = (("mixer_norm", "norm"), ("mixer", "mixer"),
                 ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))
    optional_parts = ("feed_forward_norm", "feed_forward")

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        ctx.trace("hidden_in", lambda: _hidden(stream))
        x = self.mixer_norm.forward(stream, ctx)
        ctx.trace("normed", x)
        ctx.update_into = stream
        try:
            stream.pending = self.mixer.forward(x, ctx, cache)
            if stream.pending is not None:
                ctx.trace("o", stream.pending)
            if self.feed_forward is not None:
                x = self.feed_forward_norm.forward(stream, ctx)
                ctx.trace("mlp_input", x)
                stream.pending = self.feed_forward.forward(x, ctx)
                if stream.pending is not None:
                    ctx.trace("down", stream.pending)
        finally:
            ctx.update_into = None
        ctx.trace("hidden_post_ffn", lambda: _hidden(stream))


def hidden_image(stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
    """The hidden state in the compute dtype, for a part that reads it un-normed:
    the residual itself in float32, else its rounded image (made here if nobody
    left one).  A pending update is added first."""
    if stream.pending is not None:
        stream.residual += stream.pending.float()
        stream.pending, stream.image = None, None
    if ctx.rt.dtype == torch.float32:
        return stream.residual
    if stream.image is None:
        stream.image = ctx.rt.empty(*stream.residual.shape)
        ops.round_rows(stream.residual, stream.image)
    return stream.image


@register_part("block", "output_norm")
class OutputNormBlock(Block):
    sub_parts = (("mixer_norm", "norm"), ("mixer", "mixer"),
                 ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))
    optional_parts = ("feed_forward_norm", "feed_forward")

    def __init__(self, spec):
        super().__init__(spec)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and norm.kind != "rmsnorm":
                raise ValueError(f"the output_norm block adds an rmsnorm of each sublayer's output; got a {norm.kind!r} norm")

    def _add_normed(self, update: torch.Tensor, norm, stream: ResidualStream, ctx: StepContext) -> None:
        image = None
        if ctx.rt.dtype != torch.float32:
            image = ctx.rt.empty(*stream.residual.shape)
        bias, ctx.update_bias = ctx.update_bias, None       # a bias the part left for this kernel to add
        ops.rmsnorm_add(update, norm.weight, norm.eps, stream.residual, image, bias=bias)
        stream.image = image

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        x = hidden_image(stream, ctx)
        ctx.trace("hidden_in", lambda: stream.residual.clone())
        ctx.float_updates = True
        try:
            update = self.mixer.forward(x, ctx, cache)
            ctx.trace("o", update)
            self._add_normed(update, self.mixer_norm, stream, ctx)
            if self.feed_forward is not None:
                x = hidden_image(stream, ctx)
                ctx.trace("mlp_input", x)
                update = self.feed_forward.forward(x, ctx)
                ctx.trace("down", update)
                self._add_normed(update, self.feed_forward_norm, stream, ctx)
        finally:
            ctx.float_updates = False
        ctx.trace("hidden_post_ffn", lambda: stream.residual.clone())


def _copies_sum(stream: ResidualStream) -> torch.Tensor:
    """The hidden state of a stream kept in copies, as a value (diagnostics)."""
    x = stream.copies
    if stream.pending is not None:
        mix, out_w = stream.pending_links
        x = torch.einsum("st,nsh->nth", mix, x) + out_w[None, :, None] * stream.pending.float()[:, None, :]
    return x.sum(dim=1)


@register_part("block", "hyper_connections")
class HyperConnectionsBlock(Block):
    sub_parts = (("mixer_norm", "norm"), ("mixer", "mixer"),
                 ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))
    optional_parts = ("feed_forward_norm", "feed_forward")

    def __init__(self, spec):
        super().__init__(spec)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and norm.kind != "rmsnorm":
                raise ValueError(f"the hyper_connections block reads its copies through an rmsnorm; got a {norm.kind!r} norm")
        self.hidden = int(self.param("hidden_size"))
        copies = self.p.get("copies")
        self.learned = copies is not None
        self.n_copies = int(copies) if self.learned else 1
        if not 0 < self.n_copies <= ops.HYPER_MAX_COPIES:
            raise ValueError(f"the hyper_connections block keeps 1 to {ops.HYPER_MAX_COPIES} copies, not {self.n_copies}")
        self.update_scale = float(self.p.get("update_scale") or 1.0)
        self.link_names = [str(self.param("mixer_links")) if self.learned else None,
                           str(self.param("feed_forward_links")) if self.learned and self.feed_forward is not None else None]
        self.links = [None, None]             # per sublayer: (in [S], mix [S, S], update_scale * out [S])

    def weight_specs(self) -> List[WeightSpec]:
        S, specs = self.n_copies, []
        for name in self.link_names:
            if name is not None:
                specs += [WeightSpec(name + ".in", (S,), role="parameter", mean=1.0 / S, std=0.2 / S),
                          WeightSpec(name + ".out", (S,), role="parameter", mean=1.0, std=0.2),
                          WeightSpec(name + ".mix", (S, S), role="parameter", mean=1.0 / S, std=0.2 / S)]
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        for q, name in enumerate(self.link_names):
            if name is not None:
                # the multiplier joins `out` on the host, in float64, rounded once
                out_w = (tensors[name + ".out"].to(torch.float64) * self.update_scale).to(torch.float32)
                self.links[q] = (rt.vector(tensors[name + ".in"]), rt.vector(tensors[name + ".mix"]), rt.vector(out_w))
            elif not self.learned:
                one = torch.ones(1, dtype=torch.float32)
                self.links[q] = (rt.vector(one), rt.vector(one.view(1, 1)), rt.vector(one * self.update_scale))

    def _read(self, stream: ResidualStream, ctx: StepContext, norm, in_w: torch.Tensor) -> torch.Tensor:
        """Apply what is pending, read the copies with `in_w`, norm."""
        n = stream.residual.shape[0]
        out = ctx.rt.empty(n, self.hidden)
        seed = None
        if stream.copies is None:
            # the first block of the step that keeps copies makes them from the hidden state so far
            if stream.pending is not None:
                stream.residual += stream.pending.float()
                stream.pending = None
            stream.copies = ctx.rt.empty(n, self.n_copies, self.hidden, dtype=torch.float32, lifetime="step")
            seed = stream.residual
        elif stream.copies.shape[1] != self.n_copies:
            raise ValueError(f"this layer keeps {self.n_copies} copies of the hidden state, the stream has {stream.copies.shape[1]}")
        mix, out_w = stream.pending_links if stream.pending is not None else (None, None)
        ops.hyper_norm(stream.copies, norm.weight, norm.eps, out, seed=seed, update=stream.pending, mix=mix, out_w=out_w, in_w=in_w)
        stream.pending, stream.pending_links, stream.image = None, None, None
        return out

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        in_w, mix, out_w = self.links[0]
        x = self._read(stream, ctx, self.mixer_norm, in_w)
        ctx.trace("hidden_in", lambda: _copies_sum(stream))
        ctx.trace("normed", x)
        ctx.float_updates = True
        try:
            stream.pending = self.mixer.forward(x, ctx, cache)
            stream.pending_links = (mix, out_w)
            ctx.trace("o", stream.pending)
            if self.feed_forward is not None:
                in_w, mix, out_w = self.links[1]
                x = self._read(stream, ctx, self.feed_forward_norm, in_w)
                ctx.trace("mlp_input", x)
                stream.pending = self.feed_forward.forward(x, ctx)
                stream.pending_links = (mix, out_w)
                ctx.trace("down", stream.pending)
        finally:
            ctx.float_updates = False
        ctx.trace("hidden_post_ffn", lambda: _copies_sum(stream))


@register_part("block", "concat_projection")
class ConcatProjection(Block):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.weight_name = str(self.param("weight"))
        self.source = str(self.p.get("source") or "embedding_output")
        self.w: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.hidden, 2 * self.hidden))]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.w = rt.matrix(tensors[self.weight_name])

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        kept = ctx.shared.get(self.source)
        if kept is None:
            raise ValueError(f"nothing was kept under {self.source!r} in this step for the projection to read")
        both = ctx.rt.empty(stream.residual.shape[0], 2 * self.hidden)
        ops.hidden_concat(stream.residual, stream.pending, kept, both)
        stream.pending = None
        stream.image = None
        ops.linear(both, self.w, stream.residual)
        ctx.trace("hidden_in", lambda: stream.residual.clone())
