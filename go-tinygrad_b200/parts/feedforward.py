"""Feed-forwards.

``dense``: down(act(up(x))) without a gate; ``activation`` is "relu2" (the
square of relu), "gelu_tanh" or "silu", applied in float (in bfloat16 to the
up product's float sums, in its epilogue).  Parameters:
``hidden_size``, ``intermediate_size``, ``activation`` and the tensor names
``up``, ``down``.  The reference has no ungated feed-forward.

``swiglu``: dense gated feed-forward (SwiGLU): down(silu(gate(x)) * up(x)), silu(g) =
g / (1 + exp(-g)) (model/llama.go:1361-1401, backends/simd/vec.go:52-59); with
``activation`` "gelu_tanh" or "relu2" that function stands in silu's place on the gate.

Parameters: ``hidden_size``, ``intermediate_size`` and the tensor names
``gate``, ``up``, ``down``, and optionally ``gate_bias``, ``up_bias``,
``down_bias`` (all three or none: every projection then adds its bias to its
float sums before anything else happens to them; the reference has no biases
here).  Gate and up are fused at load into one matrix
[2 * intermediate, hidden] so that one product serves both: in float32 the gate
rows come first and a second kernel applies the activation; in bfloat16 the rows
alternate in blocks of 8 gate and 8 up features and the product's epilogue
applies the activation to its float accumulators.  With biases the products
leave their float sums and two small kernels add the biases (and apply the
activation).

``routed_experts``: a mixture of `n_experts` gated silu feed-forwards without
biases, of which every token uses `top`: router logits z = R x + b in float32
(R is kept in float32), the `top` largest are the token's experts (ties: the
lower index) and their weights are the softmax over those logits alone; the
update is the weighted sum of the chosen experts' outputs.  The step's (token,
expert) pairs are ordered by expert on the device (`ops.moe_arrange`), the
experts' products run over the ordered rows, and a last kernel adds a token's
rows up in float, always in the order of its choices: no result depends on the
batch, and nothing talks to the host.  Parameters: ``hidden_size``,
``intermediate_size``, ``n_experts``, ``top``, the tensor names ``router``,
``router_bias`` (None: no bias) and ``gate``, ``up``, ``down`` with ``{e}``
standing for the expert's index.  Options: ``gate`` None makes the experts
ungated, down(act(up(x))) with ``activation`` ("relu2", "gelu_tanh", "silu");
``scoring`` "sigmoid" makes a chosen expert's weight the sigmoid of its own
logit, not renormalised (the largest sigmoids are the largest logits);
``weight_on`` "input" multiplies the expert's input by the weight instead of
its output: the update is the plain sum of expert(weight * x), the scaled rows
formed in float and rounded once.  The reference has no routed feed-forward.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import FeedForward, Runtime, StepContext, emit_update, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.names = {k: str(self.param(k)) for k in ("gate", "up", "down")}
        self.activation = str(self.p.get("activation") or "silu")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"feed-forward activation {self.activation!r} is not known; known: {sorted(ops.ACTIVATIONS)}")
        biases = [self.p.get(k) for k in ("gate_bias", "up_bias", "down_bias")]
        if any(biases) and self.activation != "silu":
            raise ValueError("a gated feed-forward with biases uses the silu activation")
        if any(biases) and not all(biases):
            raise ValueError("a gated feed-forward has biases on all three projections or on none")
        self.bias_names = [str(b) for b in biases] if all(biases) else None
        self.biases: Optional[List[torch.Tensor]] = None
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.names["gate"], (self.inter, self.hidden)),
                 WeightSpec(self.names["up"], (self.inter, self.hidden)),
                 WeightSpec(self.names["down"], (self.hidden, self.inter))]
        if self.bias_names:
            specs += [WeightSpec(name, (size,), role="parameter", std=0.02)
                      for name, size in zip(self.bias_names, (self.inter, self.inter, self.hidden))]
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        gate, up = tensors[self.names["gate"]].to(rt.dtype), tensors[self.names["up"]].to(rt.dtype)
        # bfloat16: gate and up rows interleaved in blocks of 8 so that the product's
        # epilogue can apply silu(gate) * up to its float accumulators and write the
        # activation directly; float32: gate rows then up rows, and a kernel of its own
        self.fused = (rt.dtype == torch.bfloat16 and self.inter % 8 == 0 and not self.bias_names
                      and self.activation in ops.GATED_EPILOGUES)
        if self.bias_names:
            self.biases = [rt.vector(tensors[name]) for name in self.bias_names]
        if self.fused:
            self.w_gate_up = rt.matrix(ops.interleave_gate_up(gate, up))
        else:
            self.w_gate_up = rt.matrix(torch.cat([gate, up], dim=0))
        self.w_down = rt.matrix(tensors[self.names["down"]])

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        rt = ctx.rt
        n = x.shape[0]
        if self.biases:
            return self._forward_biased(x, ctx)
        act = rt.empty(n, self.inter)
        if self.fused:
            ops.linear(x, self.w_gate_up, act, epilogue=ops.GATED_EPILOGUES[self.activation])
        else:
            gate_up = rt.empty(n, 2 * self.inter)
            ops.linear(x, self.w_gate_up, gate_up)
            ctx.trace("gate_pre", gate_up[:, : self.inter])
            ctx.trace("up", gate_up[:, self.inter:])
            ops.swiglu(gate_up, act, self.activation)
        ctx.trace("gate_act", act)
        return emit_update(act, self.w_down, ctx)


    def _forward_biased(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        rt = ctx.rt
        n = x.shape[0]
        sums = rt.empty(n, 2 * self.inter, dtype=torch.float32)
        ops.linear(x, self.w_gate_up, sums)
        act = rt.empty(n, (self.inter + 7) // 8 * 8)[:, : self.inter]
        ops.swiglu_bias(sums, self.biases[0], self.biases[1], act)
        ctx.trace("gate_act", act)
        sums = rt.empty(n, self.hidden, dtype=torch.float32)
        ops.linear(act, self.w_down, sums)
        if ctx.float_updates and ctx.op_hook is None:
            # the block's norm kernel takes float sums and adds the bias itself
            ctx.update_bias = self.biases[2]
            return sums
        out = rt.empty(n, self.hidden, dtype=torch.float32 if ctx.float_updates else None)
        ops.add_bias(sums, self.biases[2], out)
        return out


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.n_experts = int(self.param("n_experts"))
        self.top = int(self.param("top"))
        if not 0 < self.top <= self.n_experts:
            raise ValueError(f"a token cannot use {self.top} of {self.n_experts} experts")
        self.gated = self.p.get("gate") is not None
        self.activation = str(self.p.get("activation") or ("silu" if self.gated else "relu2"))
        if self.gated and self.activation != "silu":
            raise ValueError("gated experts use the silu activation")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"expert activation {self.activation!r} is not known; known: {sorted(ops.ACTIVATIONS)}")
        self.scoring = str(self.p.get("scoring") or "softmax_chosen")
        if self.scoring not in ops.MOE_SCORING:
            raise ValueError(f"router scoring {self.scoring!r} is not known; known: {sorted(ops.MOE_SCORING)}")
        self.weight_on = str(self.p.get("weight_on") or "output")
        if self.weight_on not in ("input", "output"):
            raise ValueError(f"an expert's weight multiplies its 'input' or its 'output', not {self.weight_on!r}")
        self.matrices = ("gate", "up", "down") if self.gated else ("up", "down")
        self.names = {k: str(self.param(k)) for k in ("router",) + self.matrices}
        for k in self.matrices:
            if "{e}" not in self.names[k]:
                raise ValueError(f"the experts' tensor name {self.names[k]!r} needs '{{e}}' for the expert's index")
        bias = self.p.get("router_bias")
        self.router_bias_name = str(bias) if bias else None
        self.router = self.router_bias = self.w_gate_up = self.w_down = None

    def _name(self, k: str, e: int) -> str:
        return self.names[k].replace("{e}", str(e))

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.names["router"], (self.n_experts, self.hidden))]
        if self.router_bias_name:
            specs.append(WeightSpec(self.router_bias_name, (self.n_experts,), role="parameter", std=0.02))
        for e in range(self.n_experts):
            if self.gated:
                specs.append(WeightSpec(self._name("gate", e), (self.inter, self.hidden)))
            specs += [WeightSpec(self._name("up", e), (self.inter, self.hidden)),
                      WeightSpec(self._name("down", e), (self.hidden, self.inter))]
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.router = rt.vector(tensors[self.names["router"]])
        self.router_bias = rt.vector(tensors[self.router_bias_name]) if self.router_bias_name else None
        # [E, 2I, H]: an expert's gate rows, then its up rows -- or, where the products run on the
        # tensor cores and apply the gated silu in their epilogue, alternating in blocks of 8; [E, H, I]
        self.fused = rt.dtype == torch.bfloat16 and self.inter % 8 == 0 and self.hidden % 8 == 0
        if not self.gated:
            self.w_gate_up = rt.matrix(torch.stack([tensors[self._name("up", e)].to(rt.dtype) for e in range(self.n_experts)]))
            self.w_down = rt.matrix(torch.stack([tensors[self._name("down", e)].to(rt.dtype) for e in range(self.n_experts)]))
            return
        both = (lambda g, u: ops.interleave_gate_up(g, u)) if self.fused else (lambda g, u: torch.cat([g, u], dim=0))
        self.w_gate_up = rt.matrix(torch.stack([both(tensors[self._name("gate", e)].to(rt.dtype),
                                                     tensors[self._name("up", e)].to(rt.dtype))
                                                for e in range(self.n_experts)]))
        self.w_down = rt.matrix(torch.stack([tensors[self._name("down", e)].to(rt.dtype) for e in range(self.n_experts)]))

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        rt = ctx.rt
        n, top, E = x.shape[0], self.top, self.n_experts
        chosen = rt.empty(n, top, dtype=torch.int32)
        weights = rt.empty(n, top, dtype=torch.float32)
        ops.moe_route(x, self.router, self.router_bias, chosen, weights, self.scoring)
        ctx.trace("experts", chosen)
        if not self.gated or self.weight_on == "input":
            return self._forward_general(x, ctx, chosen, weights)
        fused = self.fused and ops.moe_product_fused_supports(x, self.w_gate_up)
        # tiles of 128 rows once the experts have that many tokens each on average
        tile = 128 if fused and n * top >= 128 * E else ops.MOE_TILE_ROWS
        tiles = ops.moe_tiles_cap(n * top, E, tile)
        rows = tiles * tile
        row_item = rt.empty(rows, dtype=torch.int32)
        item_row = rt.empty(n * top, dtype=torch.int32)
        tile_expert = rt.empty(tiles, dtype=torch.int32)
        ops.moe_arrange(chosen, E, row_item, item_row, tile_expert, tile)
        act = rt.empty(rows, self.inter)
        if fused and tile == 128:
            # prompt-sized: the inputs copied into arranged order, for the product that tensor copies feed
            gathered = rt.empty(rows, self.hidden)
            ops.moe_gather(x, row_item, top, gathered)
            ops.moe_product(gathered, row_item, 0, self.w_gate_up, tile_expert, act, epilogue="swiglu")
        elif fused:
            ops.moe_product(x, row_item, top, self.w_gate_up, tile_expert, act, epilogue="swiglu")
        else:
            sums = rt.empty(rows, 2 * self.inter, dtype=torch.float32)
            ops.moe_product(x, row_item, top, self.w_gate_up, tile_expert, sums)
            ops.swiglu_bias(sums, None, None, act)
        y = rt.empty(rows, self.hidden, dtype=torch.float32)
        ops.moe_product(act, row_item, 0, self.w_down, tile_expert, y)
        out = rt.empty(n, self.hidden, dtype=torch.float32 if ctx.float_updates else None)
        ops.moe_combine(y, item_row, weights, out)
        return out


    def _forward_general(self, x: torch.Tensor, ctx: StepContext, chosen: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """Ungated experts and weights on the input: the step's (token, expert) rows are
        copied into arranged order (times their weights where those scale the input),
        and both products run over arranged rows."""
        rt = ctx.rt
        n, top, E = x.shape[0], self.top, self.n_experts
        fused = self.fused and ops.moe_product_fused_supports(x, self.w_gate_up)
        tile = 128 if fused and n * top >= 128 * E else ops.MOE_TILE_ROWS
        tiles = ops.moe_tiles_cap(n * top, E, tile)
        rows = tiles * tile
        row_item = rt.empty(rows, dtype=torch.int32)
        item_row = rt.empty(n * top, dtype=torch.int32)
        tile_expert = rt.empty(tiles, dtype=torch.int32)
        ops.moe_arrange(chosen, E, row_item, item_row, tile_expert, tile)
        on_input = self.weight_on == "input"
        gathered = rt.empty(rows, self.hidden)
        ops.moe_gather(x, row_item, top, gathered, weights=weights if on_input else None)
        act = rt.empty(rows, self.inter)
        if self.gated and fused:
            ops.moe_product(gathered, row_item, 0, self.w_gate_up, tile_expert, act, epilogue="swiglu")
        elif self.gated:
            sums = rt.empty(rows, 2 * self.inter, dtype=torch.float32)
            ops.moe_product(gathered, row_item, 0, self.w_gate_up, tile_expert, sums)
            ops.swiglu_bias(sums, None, None, act)
        else:
            ops.moe_product(gathered, row_item, 0, self.w_gate_up, tile_expert, act, epilogue=self.activation)
        ctx.trace("gate_act", act)
        y = rt.empty(rows, self.hidden, dtype=torch.float32)
        ops.moe_product(act, row_item, 0, self.w_down, tile_expert, y)
        out = rt.empty(n, self.hidden, dtype=torch.float32 if ctx.float_updates else None)
        ops.moe_combine(y, item_row, None if on_input else weights, out)
        return out


@register_part("feed_forward", "dense")
class DenseFeedForward(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.activation = str(self.p.get("activation") or "relu2")
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"feed-forward activation {self.activation!r} is not known; known: {sorted(ops.ACTIVATIONS)}")
        self.names = {k: str(self.param(k)) for k in ("up", "down")}
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.names["up"], (self.inter, self.hidden)),
                WeightSpec(self.names["down"], (self.hidden, self.inter))]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.w_up = rt.matrix(tensors[self.names["up"]])
        self.w_down = rt.matrix(tensors[self.names["down"]])

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        rt = ctx.rt
        n = x.shape[0]
        act = rt.empty(n, (self.inter + 7) // 8 * 8)[:, : self.inter]
        if ctx.op_hook is None:
            # the activation rides in the product's epilogue, on its float sums, where the kernel has one
            ops.linear(x, self.w_up, act, epilogue=self.activation)
        else:
            ops.linear(x, self.w_up, act)
            ctx.trace("up", lambda: act.clone())
            ops.activation(act, self.activation)
        ctx.trace("gate_act", act)
        return emit_update(act, self.w_down, ctx)
