"""Token embedding and the output head.

``token_embedding``: x = E[token] (unscaled: model/inference_helpers.go:9-34),
or E[token] * ``scale`` where a scale is given;
it starts the float32 residual stream.  Parameters: ``vocab_size``,
``hidden_size``, ``weight`` and optionally ``scale``, ``position`` (a position PartSpec
whose `on_embedding` hook acts on the embedded tokens), ``keep_output``
(True: a float32 copy of the embedded tokens stays in the step's shared values
as "embedding_output" for later parts to read) and ``norm`` ({"weight": tensor
name, "eps": e}: the embedded tokens pass an RMS norm with that weight, in
float32, and the normed rows are the hidden state the first layer adds to).

``lm_head``: logits = x . LM^T in float32 for the rows it is given
(model/inference_helpers.go:122-148).  ``weight`` names the table; with
``tied`` it is the embedding's tensor and one device copy serves both
(model/llama.go:490-494 decides tying by the tensor's presence; here the
configuration's flag decides and a stray ``ignored`` tensor is tolerated).
With ``softcap`` c the logits become c * tanh(logits / c); with ``scale`` m they
are multiplied by m (after the cap, if there is one).
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import (Embedding, Head, ResidualStream, Runtime, StepContext, build_part,
                   register_part)


@register_part("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.weight_name = str(self.param("weight"))
        pos = self.p.get("position")
        self.position = build_part("position", pos) if pos is not None else None
        self.keep_output = bool(self.p.get("keep_output", False))
        self.scale = float(self.p.get("scale") or 1.0)
        norm = self.p.get("norm")
        self.norm_name = str(norm["weight"]) if norm else None
        self.norm_eps = float(norm["eps"]) if norm else 0.0
        self.norm_weight: Optional[torch.Tensor] = None
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.weight_name, (self.vocab, self.hidden), role="table")]
        if self.norm_name:
            specs.append(WeightSpec(self.norm_name, (self.hidden,), role="vector", mean=1.0))
        return specs

    def children(self):
        return [self.position] if self.position else []

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.table = rt.matrix(tensors[self.weight_name], share_as=self.weight_name)
        if self.norm_name:
            self.norm_weight = rt.vector(tensors[self.norm_name])

    def forward(self, ctx: StepContext) -> ResidualStream:
        residual = ctx.rt.empty(ctx.n_tokens, self.hidden, dtype=torch.float32, lifetime="step")
        ops.embed(ctx.tokens, self.table, residual, self.scale)
        if self.norm_weight is not None:
            ops.rmsnorm_rows(residual, self.norm_weight, self.norm_eps)
        if self.keep_output:
            kept = ctx.rt.empty(ctx.n_tokens, self.hidden, dtype=torch.float32, lifetime="step")
            ops.embed(ctx.tokens, self.table, kept, self.scale)
            ctx.shared["embedding_output"] = kept
        stream = ResidualStream(residual)
        if self.position:
            self.position.on_embedding(stream, ctx)
        return stream


@register_part("head", "lm_head")
class LMHead(Head):
    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.weight_name = str(self.param("weight"))
        self.tied = bool(self.p.get("tied", False))
        self.ignored = self.p.get("ignored")
        cap = self.p.get("softcap")
        self.softcap = float(cap) if cap else None
        scale = self.p.get("scale")
        self.scale = float(scale) if scale is not None and float(scale) != 1.0 else None
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.weight_name, (self.vocab, self.hidden), role="table")]
        if self.ignored:
            specs.append(WeightSpec(str(self.ignored), (self.vocab, self.hidden), role="ignored",
                                    optional=True))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.table = rt.matrix(tensors[self.weight_name], share_as=self.weight_name)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        logits = ctx.rt.result(x.shape[0], self.vocab, dtype=torch.float32)
        ops.linear(x, self.table, logits)
        if self.softcap:
            ops.softcap(logits, self.softcap)
        if self.scale is not None:
            ops.scale(logits, self.scale)
        return logits
