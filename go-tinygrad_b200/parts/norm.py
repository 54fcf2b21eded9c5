"""Norms, fused with the residual add that precedes them.

``rmsnorm``: y = w * x * (1/sqrt(mean(x^2) + eps)) with the sum of squares and
the scale in float32 (backends/simd/vec.go:72-85).  Parameters: ``size``,
``eps``, ``weight`` (tensor name).

Handed a stream whose hidden state is kept in several copies
(`ResidualStream.copies`), ``rmsnorm`` norms their sum and applies a pending
update by its links on the way.

``layernorm``: y = (x - mean(x)) / sqrt(var(x) + eps) * w + b, var the mean of
the squared deviations, all in float32.  Parameters: ``size``, ``eps``,
``weight`` and ``bias`` (tensor names; ``bias`` None for a norm without one).
The reference has no such norm.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Norm, ResidualStream, Runtime, StepContext, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))
        self.weight_name = str(self.param("weight"))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.size,), role="vector", mean=1.0)]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = rt.vector(tensors[self.weight_name])

    def forward(self, stream: ResidualStream, ctx: StepContext,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n_out = rows.numel() if rows is not None else stream.residual.shape[0]
        out = ctx.rt.empty(n_out, self.size)
        if stream.copies is not None:
            # the hidden state is the sum of its copies; a pending update joins them by its links first
            mix, out_w = stream.pending_links if stream.pending is not None else (None, None)
            ops.hyper_norm(stream.copies, self.weight, self.eps, out, update=stream.pending, mix=mix, out_w=out_w, rows=rows)
            if rows is None:
                stream.pending, stream.pending_links, stream.image = None, None, None
            return out
        ops.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out, rows)
        if rows is None:
            if stream.pending is not None:
                stream.image = None
            stream.pending = None
        return out


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))
        self.weight_name = str(self.param("weight"))
        bias = self.p.get("bias")
        self.bias_name = str(bias) if bias else None
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.weight_name, (self.size,), role="vector", mean=1.0)]
        if self.bias_name:
            specs.append(WeightSpec(self.bias_name, (self.size,), role="vector", mean=0.0))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.weight = rt.vector(tensors[self.weight_name])
        self.bias = rt.vector(tensors[self.bias_name]) if self.bias_name else None

    def forward(self, stream: ResidualStream, ctx: StepContext,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n_out = rows.numel() if rows is not None else stream.residual.shape[0]
        out = ctx.rt.empty(n_out, self.size)
        ops.add_layernorm(stream.residual, stream.pending, self.weight, self.bias, self.eps, out, rows)
        if rows is None:
            if stream.pending is not None:
                stream.image = None
            stream.pending = None
        return out
