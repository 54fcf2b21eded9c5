"""Grouped-query attention with a position encoding on queries and keys.

q, k, v = x Wq^T, x Wk^T, x Wv^T; rotate q and k; store k (after rotation) and
v in the cache; per query head h, softmax((q_h . K_{h // group}) * scale) V,
causal within the sequence, optionally over the last `window` keys only; then
the output projection (model/llama.go:1111-1137 projections, :1230-1233
rotation, :1253-1254 cache write, :1603-1661 attention, :1290-1297 output).

Parameters: ``hidden_size``, ``n_heads``, ``n_kv_heads``, ``head_dim``,
``window`` (None: all keys), ``scale`` (None: head_dim^-1/2), ``position`` (a
position PartSpec), ``own_kv`` (False for a layer that has no key/value
projections and reads another run's cache), ``values`` ("projection", the
default, or "keys": there is no value projection and the value of a token is
its key as projected, before the rotation), and the tensor names ``q``, ``k``,
``v``, ``o``.  The projections are fused at load into one matrix
[(n_heads + 2 n_kv_heads) * head_dim, hidden] (without the value rows when the
values are the keys) so that one product serves them.

Further options, none of which the reference has; a mixer that uses any of them
takes the general route (`_forward_general`): the fused projection leaves float
sums, one kernel finishes them (`ops.qkv_finish`: biases, rotation, unit norm,
value blend, gate, cache store, all in float and rounded once), and the
attention kernels that know the options follow.
``value_dim``: channels of a value head where they differ from a key head's
(the cache then keeps value rows of that width, the output projection reads
n_heads * value_dim columns).  ``q_bias``, ``k_bias``, ``v_bias``: tensor names
of biases added in the projection (all three or none).  ``qk_norm`` "unit":
after the rotation every query and key head is divided by its root mean square
over the head, x / sqrt(mean(x^2) + ``norm_eps``), without a weight.  ``chunk``:
positions are cut into stretches of so many, counted from the sequence's first
token, and a query sees the keys at or before it within its own stretch only.
``head_gate``: tensor name [n_heads, hidden]; head h's output is multiplied by
sigmoid(gate_h . x) before the output projection.  ``value_blend``: {"role":
"source" | "blend", "weight": tensor name of a scalar, "key": a name}: the
"source" layer leaves its values for the step under the key, a "blend" layer
caches and attends (1 - w) v + w v_source for the same token (the source's own
scalar exists in the checkpoint and is not read).

A second family of options, which go together and not with the ones above
except ``value_dim`` and the biases (`_forward_conv`; `ops.qkv_conv_finish` stands
between projection and attention).  ``conv``: {"taps": n, "q": name, "k": name,
"v": name}, tensors [channels, taps] whose last column is the current token's:
every channel of the biased q, k and v passes a causal convolution over the last
n tokens, zeros before the sequence's start, directly behind the projection; the
sequence's last n - 1 projected rows are kept as per-sequence state.
``qk_norm`` "weight" with ``q_norm`` and ``k_norm`` (tensor names, [head_dim]):
an RMS norm with that weight on every query and key head, before the rotation,
eps ``norm_eps``.  A position encoding with interleaved pairs.  ``softcap`` c:
scores become c tanh(score / c) after the scale.  ``output_gate``: tensor name
[n_heads * value_dim, hidden]; the concatenated heads are multiplied channel by
channel by sigmoid(G x) before the output projection.  With ``own_kv`` False the
layer has none of the key and value tensors and reads another run's cache with
queries, convolution state, window and gate of its own.  ``cache_window`` (where
given): how many keys the cache keeps for this layer's storage instead of
``window`` (None: all of them): a layer whose keys other layers read through
longer windows, or through none, must keep what the longest-sighted of them sees.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..cache import CacheHandle, KVRequest, Request, StateRequest
from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Mixer, Runtime, StepContext, build_part, emit_update, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.n_kv = int(self.param("n_kv_heads"))
        self.head_dim = int(self.param("head_dim"))
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} query heads cannot share {self.n_kv} key/value heads")
        window = self.p.get("window")
        self.window = int(window) if window else None
        kept = self.p["cache_window"] if "cache_window" in self.p else window
        self.cache_window = int(kept) if kept else None
        if self.cache_window is not None and (self.window is None or self.cache_window < self.window):
            raise ValueError(f"a cache that keeps {self.cache_window} keys cannot serve a window of {self.window or 'all'}")
        scale = self.p.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.own_kv = bool(self.p.get("own_kv", True))
        self.values = str(self.p.get("values") or "projection")
        if self.values not in ("projection", "keys"):
            raise ValueError(f"attention values {self.values!r} are not known: 'projection' or 'keys'")
        self.v_from_k = self.values == "keys"
        self.position = build_part("position", self.param("position"))
        wanted = ("q", "o") if not self.own_kv else ("q", "k", "o") if self.v_from_k else ("q", "k", "v", "o")
        self.names = {k: str(self.param(k)) for k in wanted}
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv * self.head_dim
        # ---- options of the general route
        self.value_dim = int(self.p.get("value_dim") or self.head_dim)
        self.v_width = self.n_kv * self.value_dim
        biases = [self.p.get(k) for k in (("q_bias", "k_bias", "v_bias") if self.own_kv else ("q_bias",))]
        if any(biases) and not all(biases):
            raise ValueError("an attention mixer has biases on q, k and v or on none of them")
        self.bias_names = [str(b) for b in biases] if all(biases) else None
        self.qk_norm = self.p.get("qk_norm")
        if self.qk_norm not in (None, "unit", "weight"):
            raise ValueError(f"qk_norm {self.qk_norm!r} is not known: None, 'unit' or 'weight'")
        conv = self.p.get("conv")
        self.conv = dict(conv) if conv and int(conv.get("taps", 0)) > 0 else None
        self.taps = int(self.conv["taps"]) if self.conv else 1
        cap = self.p.get("softcap")
        self.softcap = float(cap) if cap else 0.0
        out_gate = self.p.get("output_gate")
        self.out_gate_name = str(out_gate) if out_gate else None
        self.conv_route = bool(self.conv or self.qk_norm == "weight" or self.softcap or self.out_gate_name
                               or self.position.pairing == "interleaved")
        self.norm_eps = float(self.p.get("norm_eps") or 0.0)
        chunk = self.p.get("chunk")
        self.chunk = int(chunk) if chunk else None
        gate = self.p.get("head_gate")
        self.gate_name = str(gate) if gate else None
        blend = self.p.get("value_blend")
        self.blend = dict(blend) if blend else None
        if self.blend and self.blend.get("role") not in ("source", "blend"):
            raise ValueError(f"value_blend role {self.blend.get('role')!r} is not known: 'source' or 'blend'")
        self.general = bool(self.value_dim != self.head_dim or self.bias_names or self.qk_norm or self.chunk
                            or self.gate_name or self.blend or self.conv_route)
        if self.conv_route and (self.qk_norm == "unit" or self.chunk or self.gate_name or self.blend or self.v_from_k):
            raise ValueError("convolved projections, weighted head norms, capped scores and the gate on all channels are "
                             "not built together with unit norms, stretches of keys, gates per head or blended values")
        if self.general and (self.v_from_k or (not self.own_kv and not self.conv_route)):
            raise ValueError("the options of the general attention route need key and value projections of the layer's own")
        self.norm_names = None
        if self.qk_norm == "weight":
            self.norm_names = [str(self.param("q_norm"))] + ([str(self.param("k_norm"))] if self.own_kv else [])
        # channels that pass the convolution: q, and k and v where the layer has them
        self.conv_channels = self.q_dim + ((self.kv_dim + self.v_width) if self.own_kv else 0)
        self.conv_w = self.q_norm_w = self.k_norm_w = None
        self.bias: Optional[torch.Tensor] = None
        self.blend_weight = 0.0
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.names["q"], (self.q_dim, self.hidden))]
        if self.own_kv:
            specs.append(WeightSpec(self.names["k"], (self.kv_dim, self.hidden)))
            if not self.v_from_k:
                specs.append(WeightSpec(self.names["v"], (self.v_width, self.hidden)))
        specs.append(WeightSpec(self.names["o"], (self.hidden, self.n_heads * self.value_dim)))
        if self.bias_names:
            specs += [WeightSpec(name, (size,), role="parameter", std=0.02)
                      for name, size in zip(self.bias_names, (self.q_dim, self.kv_dim, self.v_width))]
        if self.conv:
            specs += [WeightSpec(str(self.conv[k]), (size, self.taps), role="parameter", mean=1.0 / self.taps, std=0.3)
                      for k, size in self._conv_parts()]
        if self.norm_names:
            specs += [WeightSpec(name, (self.head_dim,), role="vector", mean=1.0) for name in self.norm_names]
        if self.out_gate_name:
            specs.append(WeightSpec(self.out_gate_name, (self.n_heads * self.value_dim, self.hidden)))
        if self.gate_name:
            specs.append(WeightSpec(self.gate_name, (self.n_heads, self.hidden)))
        if self.blend:
            source = self.blend["role"] == "source"
            specs.append(WeightSpec(str(self.blend["weight"]), (), role="ignored" if source else "parameter",
                                    optional=source, mean=0.3, std=0.1))
        return specs

    def _conv_parts(self):
        parts = [("q", self.q_dim)]
        if self.own_kv:
            parts += [("k", self.kv_dim), ("v", self.v_width)]
        return parts

    def children(self):
        return [self.position]

    def cache_requests(self) -> List[Request]:
        if self.conv_route:
            requests: List[Request] = []
            if self.own_kv:
                requests.append(KVRequest(self.n_kv, self.head_dim, self.cache_window, value_dim=self.value_dim))
            if self.taps > 1:
                requests.append(StateRequest("conv", (self.taps - 1, self.conv_channels), "float32"))
            return requests
        if not self.own_kv:
            return []
        if self.general:
            return [KVRequest(self.n_kv, self.head_dim, self.cache_window, value_dim=self.value_dim, chunk=self.chunk)]
        return [KVRequest(self.n_kv, self.head_dim, self.cache_window)]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        parts = [tensors[self.names["q"]]]
        if self.own_kv:
            parts.append(tensors[self.names["k"]])
            if not self.v_from_k:
                parts.append(tensors[self.names["v"]])
        if self.gate_name:
            parts.append(tensors[self.gate_name])
        if self.out_gate_name:
            parts.append(tensors[self.out_gate_name])
        rows = sum(p.shape[0] for p in parts)
        if self.general and rows % 8:
            # whole groups of 8 rows, so that the products' float sums keep rows of a multiple of 32 bytes
            parts.append(torch.zeros((8 - rows % 8, self.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.w_qkv = rt.matrix(torch.cat([p.to(rt.dtype) for p in parts], dim=0))
        self.w_o = rt.matrix(tensors[self.names["o"]])
        if self.bias_names:
            self.bias = rt.vector(torch.cat([tensors[name].reshape(-1).to(torch.float32) for name in self.bias_names]))
        if self.blend and self.blend["role"] == "blend":
            self.blend_weight = float(tensors[str(self.blend["weight"])].to(torch.float32))
        if self.conv:
            # tap by tap, [taps, q | k | v]: neighbouring channels read neighbouring weights
            self.conv_w = rt.vector(torch.cat([tensors[str(self.conv[k])].to(torch.float32) for k, _ in self._conv_parts()],
                                              dim=0).t().contiguous())
        if self.norm_names:
            self.q_norm_w = rt.vector(tensors[self.norm_names[0]])
            self.k_norm_w = rt.vector(tensors[self.norm_names[1]]) if self.own_kv else None

    def _forward_conv(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        kv = cache.kv
        n = x.shape[0]
        sums = rt.empty(n, self.w_qkv.shape[0], dtype=torch.float32)
        ops.linear(x, self.w_qkv, sums)
        rotation = self.position.rotation(ctx)
        q = rt.empty(n, self.q_dim)
        state = cache.state("conv") if self.taps > 1 else None
        ops.qkv_conv_finish(sums, self.bias, self.conv_w, state, ctx.cu_seqlens, self.q_norm_w, self.k_norm_w, self.norm_eps,
                            rotation, self.position.pairing == "interleaved", self.n_heads, self.n_kv if self.own_kv else 0,
                            self.head_dim, self.value_dim, kv, q, ctx.token_seq, ctx.slots, ctx.positions,
                            store=cache.writes and self.own_kv, one_token_each=ctx.is_decode)
        if state is not None:
            # the convolution has read what it needed of the old state: now the step's raw sums join it
            ops.conv_state_update(sums[:, : self.conv_channels], state, ctx.cu_seqlens, ctx.slots, ctx.n_seqs)
        ctx.trace("q_attn", q)
        mixed = rt.empty(n, self.n_heads * self.value_dim)
        logits = sums[:, self.conv_channels: self.conv_channels + self.n_heads * self.value_dim] if self.out_gate_name else None
        ops.attention_general(q, mixed, kv, ctx, self.n_heads, self.scale, window=self.window or 0,
                              softcap=self.softcap, gate_logits=logits)
        ctx.trace("attn", mixed)
        return emit_update(mixed, self.w_o, ctx)

    def _forward_general(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        kv = cache.kv
        n = x.shape[0]
        sums = rt.empty(n, self.w_qkv.shape[0], dtype=torch.float32)
        ops.linear(x, self.w_qkv, sums)
        rotation = self.position.rotation(ctx)
        if rotation is not None and self.position.pairing != "half":
            raise ValueError("the general attention route rotates half-split pairs only")
        q = rt.empty(n, self.q_dim)
        gate = rt.empty(n, self.n_heads, dtype=torch.float32) if self.gate_name else None
        v_first = v_keep = None
        if self.blend:
            key = ("value_blend", self.blend.get("key"))
            if self.blend["role"] == "source":
                v_keep = rt.empty(n, self.v_width, dtype=torch.float32, lifetime="step")
                ctx.shared[key] = v_keep
            else:
                v_first = ctx.shared.get(key)
                if v_first is None or tuple(v_first.shape) != (n, self.v_width):
                    raise ValueError("no layer of this step has left values of this layer's shape to blend with")
        ops.qkv_finish(sums, self.bias, rotation, self.n_heads, kv, q, ctx.token_seq, ctx.slots, ctx.positions,
                       unit_norm=self.qk_norm == "unit", eps=self.norm_eps, v_first=v_first, v_keep=v_keep,
                       blend=self.blend_weight, gate_out=gate, store=cache.writes)
        ctx.trace("q_attn", q)
        mixed = rt.empty(n, self.n_heads * self.value_dim)
        ops.attention_general(q, mixed, kv, ctx, self.n_heads, self.scale, window=self.window or 0,
                              chunk=self.chunk or 0, gate=gate)
        ctx.trace("attn", mixed)
        if ctx.float_updates:
            out = rt.empty(n, self.hidden, dtype=torch.float32)
            ops.linear(mixed, self.w_o, out)
            return out
        return emit_update(mixed, self.w_o, ctx)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        kv = cache.kv
        if kv is None or kv.n_kv_heads != self.n_kv or kv.head_dim != self.head_dim or kv.value_dim != self.value_dim:
            raise ValueError("attention was given a cache entry that does not match its heads")
        if self.conv_route:
            return self._forward_conv(x, ctx, cache)
        if self.general:
            return self._forward_general(x, ctx, cache)
        n = x.shape[0]
        qkv = rt.empty(n, self.w_qkv.shape[0])
        rotation = self.position.rotation(ctx)
        pairing, rotary_dim = self.position.pairing, self.position.rotary_dim or self.head_dim
        # the kernels that rotate inside a product or inside the attention know one
        # layout: half-split pairs over the whole head; any other goes the general way
        plain_layout = rotation is None or (pairing == "half" and rotary_dim == self.head_dim)
        store = self.n_kv if (cache.writes and self.own_kv) else 0
        # a decode step in bfloat16: the attention kernel rotates the queries and adds the new
        # token's key and value itself, and no kernel stands between it and the projection
        in_attention = (ctx.is_decode and rt.dtype == torch.bfloat16 and plain_layout
                        and ops.attention_bf16_supports(self.head_dim))
        if store and plain_layout and not self.v_from_k and ops.qkv_rope_fused_supports(x, self.w_qkv, qkv, rotation, self.n_heads,
                                                                  self.n_kv, self.head_dim, kv):
            # a prompt: rotation and cache store happen in the projection's epilogue
            ops.linear_qkv_rope(x, self.w_qkv, qkv, rotation, self.n_heads, self.n_kv, kv,
                                ctx.token_seq, ctx.slots, ctx.positions)
            in_attention = False
        else:
            ops.linear(x, self.w_qkv, qkv)
            if ctx.op_hook is not None:
                ctx.trace("q", qkv[:, : self.q_dim].clone())
                if self.own_kv:
                    ctx.trace("k", qkv[:, self.q_dim: self.q_dim + self.kv_dim])
                    ctx.trace("v", qkv[:, self.q_dim + (0 if self.v_from_k else self.kv_dim):][:, : self.kv_dim])
            if not in_attention:
                ops.rope_kv_store(qkv, rotation, self.n_heads, store, self.head_dim,
                                  kv, ctx.token_seq, ctx.slots, ctx.positions,
                                  pairing=pairing, rotary_dim=rotary_dim, values_from_keys=self.v_from_k)
        q = qkv[:, : self.q_dim]
        if not in_attention:
            ctx.trace("q_attn", q)
        mixed = rt.empty(n, self.q_dim)
        window = self.window or 0
        if rt.dtype == torch.bfloat16 and ops.attention_bf16_supports(self.head_dim):
            if ctx.is_decode:
                new_k = qkv[:, self.q_dim: self.q_dim + self.kv_dim] if store else None
                new_v = (new_k if self.v_from_k else qkv[:, self.q_dim + self.kv_dim:]) if store else None
                splits, chunk, ring = ops.attention_decode_plan(n, self.n_heads, self.n_kv, self.head_dim,
                                                          ctx.max_kv_len, window, ctx.total_kv_len)
                scratch = None
                if splits > 1:
                    scratch = rt.empty(ops.attention_decode_scratch_floats(
                        n, self.n_heads, self.head_dim, splits), dtype=torch.float32)
                ops.attention_decode_bf16(q, mixed, kv, ctx.slots, ctx.positions, self.n_heads,
                                          self.scale, window, splits, scratch,
                                          unrotated=(rotation, new_k, new_v, True) if in_attention else None,
                                          chunk_pages=chunk, ring_pages=ring)
            elif ops.attention_tcgen05_supports(kv) and qkv.stride(0) % 8 == 0:
                ops.attention_prefill_tcgen05(q, mixed, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos,
                                              ctx.n_seqs, ctx.max_q_len, self.n_heads, self.scale, window)
            else:
                ops.attention_prefill_bf16(q, mixed, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos,
                                           ctx.n_seqs, ctx.max_q_len, self.n_heads, self.scale, window)
        else:
            ops.attention_simple(q, mixed, kv, ctx.token_seq, ctx.slots, ctx.positions,
                                 self.n_heads, self.scale, window)
        ctx.trace("attn", mixed)
        return emit_update(mixed, self.w_o, ctx)
