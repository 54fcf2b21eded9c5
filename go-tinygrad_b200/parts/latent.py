"""Attention through a latent.

A token keeps, instead of keys and values per head, one latent vector c of
``kv_rank`` channels (a down projection of the mixer's input, RMS-normed with a
weight of its own) and one rotated key part of ``rot_dim`` channels that all
heads share (further rows of the same down projection, not normed).  Head h has
a query [a_h | b_h] of ``head_dim`` unrotated and ``rot_dim`` rotated channels,
an unrotated key U_h c and a value V_h c; its score against an earlier token is
(a_h . U_h c + b_h' . k') * scale (' = rotated), seen through a causal window.
The heads, side by side, are multiplied by sigmoid(G x) where the part has a
gate, and projected by O.  The reference has no such mixer.

What runs: one product gives q, the gate and the down projection; one kernel
norms the latent, rotates the shared key part, stores both in the token's cache
row [c | k'] and rotates the b_h; a product per head folds U_h into the query,
a_h -> U_h^T a_h, so that query rows [U_h^T a_h | b_h'] meet cache rows directly
(a_h . U_h c = U_h^T a_h . c); attention then runs over one shared key/value
head of kv_rank + rot_dim channels whose values are its first kv_rank channels;
a product per head applies V_h to the attended latents.  The cache holds
kv_rank + rot_dim numbers a token and one plane, whatever the head count.

A step whose sequences all start at their first token (whole prompts, in
bfloat16) takes another road after the per-token kernel: its own rows are all
the keys there are, so one product expands them per head (U_h c and V_h c for
all heads) and attention runs over those, dim + rot channels a score and v_dim a
value instead of kv_rank + rot_dim and kv_rank.  The layer with the down
projection leaves the step's rows in the step's shared values for the layers
that read its cache.

Parameters: ``hidden_size``, ``n_heads``, ``head_dim``, ``rot_dim``, ``v_dim``,
``kv_rank``, ``window`` (None: all keys), ``scale`` (None: (head_dim +
rot_dim)^-1/2), ``eps`` (of the latent's norm), ``position`` (a rotary
PartSpec over the rotated part: interleaved pairs; it may rotate fewer
channels than rot_dim), ``own_kv`` (False: no down projection, the run reads
another run's cache rows), and the tensor names ``q``, ``dkv``, ``dkv_norm``,
``uk``, ``uv``, ``gate`` (None: no gate), ``o``.  Options: the position part may
pair channel i with i + rot.dims/2 instead ("half"); ``q_latent`` ({"rank": r,
"down": name, "norm": name}): the queries come through a latent of their own,
q = W_q rmsnorm(W_down x) with that norm's weight and ``eps``, and ``q`` is then
[heads * (head_dim + rot_dim), r]; ``sinks`` (tensor name, [heads]): exp(sink_h)
joins head h's softmax denominator, without a key or a value and unscaled.
"""
from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..cache import CacheHandle, KVRequest, Request
from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Mixer, Runtime, StepContext, build_part, emit_update, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.dim = int(self.param("head_dim"))
        self.rot = int(self.param("rot_dim"))
        self.v_dim = int(self.param("v_dim"))
        self.rank = int(self.param("kv_rank"))
        window = self.p.get("window")
        self.window = int(window) if window else None
        scale = self.p.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.dim + self.rot)
        self.eps = float(self.param("eps"))
        self.own_kv = bool(self.p.get("own_kv", True))
        self.position = build_part("position", self.param("position"))
        if (self.position.rotary_dim or self.rot) > self.rot:
            raise ValueError("latent attention rotates pairs within its rotated part")
        if self.rot % 2:
            raise ValueError(f"the rotated part needs an even number of channels, got {self.rot}")
        wanted = ["q", "uk", "uv", "o"] + (["dkv", "dkv_norm"] if self.own_kv else [])
        self.names = {k: str(self.param(k)) for k in wanted}
        gate = self.p.get("gate")
        if gate:
            self.names["gate"] = str(gate)
        q_latent = self.p.get("q_latent")
        self.q_rank = int(q_latent["rank"]) if q_latent else 0
        if q_latent:
            self.names["q_down"], self.names["q_norm"] = str(q_latent["down"]), str(q_latent["norm"])
        sinks = self.p.get("sinks")
        if sinks:
            self.names["sinks"] = str(sinks)
        self.sinks = self.w_q_down = self.w_q_up = self.q_norm_w = None
        self.row = self.rank + self.rot                     # a cache row, and a folded query row of a head
        self.q_dim = self.n_heads * (self.dim + self.rot)
        self.g_dim = self.n_heads * self.v_dim if gate else 0
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.norm_w = self.w_expand = None

    def weight_specs(self) -> List[WeightSpec]:
        H = self.n_heads
        specs = [WeightSpec(self.names["q"], (self.q_dim, self.q_rank or self.hidden))]
        if self.q_rank:
            specs += [WeightSpec(self.names["q_down"], (self.q_rank, self.hidden)),
                      WeightSpec(self.names["q_norm"], (self.q_rank,), role="vector", mean=1.0)]
        if "sinks" in self.names:
            specs.append(WeightSpec(self.names["sinks"], (H,), role="parameter", std=1.0))
        if self.own_kv:
            specs += [WeightSpec(self.names["dkv"], (self.row, self.hidden)),
                      WeightSpec(self.names["dkv_norm"], (self.rank,), role="vector", mean=1.0)]
        specs += [WeightSpec(self.names["uk"], (H * self.dim, self.rank)),
                  WeightSpec(self.names["uv"], (H * self.v_dim, self.rank))]
        if "gate" in self.names:
            specs.append(WeightSpec(self.names["gate"], (H * self.v_dim, self.hidden)))
        specs.append(WeightSpec(self.names["o"], (self.hidden, H * self.v_dim)))
        return specs

    def children(self):
        return [self.position]

    def cache_requests(self) -> List[Request]:
        return [KVRequest(1, self.row, self.window, planes=1)] if self.own_kv else []

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        H = self.n_heads
        parts = [] if self.q_rank else [tensors[self.names["q"]]]
        if self.q_rank:
            self.w_q_down = rt.matrix(tensors[self.names["q_down"]])
            self.w_q_up = rt.matrix(tensors[self.names["q"]])
            self.q_norm_w = rt.vector(tensors[self.names["q_norm"]])
        if "sinks" in self.names:
            self.sinks = rt.vector(tensors[self.names["sinks"]].reshape(-1))
        if "gate" in self.names:
            parts.append(tensors[self.names["gate"]])
        if self.own_kv:
            parts.append(tensors[self.names["dkv"]])
            self.norm_w = rt.vector(tensors[self.names["dkv_norm"]])
        self.w_in = rt.matrix(torch.cat([p.to(rt.dtype) for p in parts], dim=0)) if parts else None
        # U_h^T per head, [H, rank, dim]: the product that folds U_h into the query reads it as its weight
        self.w_uk_t = rt.matrix(tensors[self.names["uk"]].to(rt.dtype).reshape(H, self.dim, self.rank).transpose(1, 2))
        self.w_uv = rt.matrix(tensors[self.names["uv"]]).view(H, self.v_dim, self.rank)
        # per head [U_h; V_h; rot_dim rows of zeros], [H * (dim + v_dim + rot_dim), rank]: the product that expands a
        # prompt's rows into one run per token and head, with room for the rotated key part behind key and value
        self.w_expand = None
        if rt.dtype == torch.bfloat16:
            uk = tensors[self.names["uk"]].to(rt.dtype).reshape(H, self.dim, self.rank)
            uv = tensors[self.names["uv"]].to(rt.dtype).reshape(H, self.v_dim, self.rank)
            room = torch.zeros(H, self.rot, self.rank, dtype=rt.dtype, device=uk.device)   # tensors come from a file or, random, from the device
            self.w_expand = rt.matrix(torch.cat([uk, uv, room], dim=1).reshape(-1, self.rank))
        self.w_o = rt.matrix(tensors[self.names["o"]])

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        kv = cache.kv
        if kv is None or kv.n_kv_heads != 1 or kv.head_dim != self.row:
            raise ValueError("latent attention was given a cache entry that does not hold its rows")
        n, H = x.shape[0], self.n_heads
        width = self.w_in.shape[0] if self.w_in is not None else 0
        proj = rt.empty(n, (width + 7) // 8 * 8)[:, :width] if width else None
        if width:
            ops.linear(x, self.w_in, proj)
        if self.q_rank:
            # queries through their own latent: the down projection leaves float sums, the norm reads those
            q_sums = rt.empty(n, self.q_rank, dtype=torch.float32)
            ops.linear(x, self.w_q_down, q_sums)
            cq = rt.empty(n, self.q_rank)
            ops.add_rmsnorm(q_sums, None, self.q_norm_w, self.eps, cq)
            q = rt.empty(n, (self.q_dim + 7) // 8 * 8)[:, : self.q_dim]
            ops.linear(cq, self.w_q_up, q)
            q_cols = 0
        else:
            q = proj[:, : self.q_dim]
            q_cols = self.q_dim
        gate = proj[:, q_cols: q_cols + self.g_dim] if self.g_dim else None
        dkv = proj[:, q_cols + self.g_dim:] if (self.own_kv and cache.writes) else None
        rotation = self.position.rotation(ctx)
        pairing = self.position.pairing
        if self._expands(ctx, cache):
            return self._forward_expanded(x, ctx, cache, q, gate, dkv, rotation)
        folded = rt.empty(n, H * self.row)
        ops.latent_prepare(q, dkv, rotation, self.norm_w, self.eps, kv, ctx.token_seq, ctx.slots, ctx.positions,
                           folded, H, self.dim, self.rot, self.rank, pairing=pairing)
        ops.linear_heads(q.view(n, H, self.dim + self.rot)[:, :, : self.dim], self.w_uk_t,
                         folded.view(n, H, self.row)[:, :, : self.rank])
        ctx.trace("q_attn", folded)
        attended = rt.empty(n, H * self.rank)
        if rt.dtype == torch.bfloat16 and ops.latent_attention_supports(kv, self.rank):
            splits, floats = ops.latent_attention_plan(ctx.n_seqs, ctx.max_q_len, H, self.row, self.rank, ctx.max_kv_len,
                                                       self.window or 0)
            scratch = rt.empty(n * floats, dtype=torch.float32) if splits > 1 else None
            ops.latent_attention_bf16(folded, attended, kv, ctx.cu_seqlens, ctx.slots, ctx.start_pos, ctx.n_seqs,
                                      ctx.max_q_len, H, self.rank, self.scale, self.window or 0, splits, scratch,
                                      sinks=self.sinks)
        else:
            # float32, and row sizes the tensor-core kernel does not take
            ops.attention_simple(folded, attended, kv, ctx.token_seq, ctx.slots, ctx.positions, H, self.scale,
                                 self.window or 0, value_dim=self.rank, sinks=self.sinks)
        heads = rt.empty(n, (H * self.v_dim + 7) // 8 * 8)[:, : H * self.v_dim]
        ops.linear_heads(attended.view(n, H, self.rank), self.w_uv, heads.view(n, H, self.v_dim),
                         gate.view(n, H, self.v_dim) if gate is not None else None)
        ctx.trace("attn", heads)
        return emit_update(heads, self.w_o, ctx)

    # ------------------------------------------------- whole prompts: keys and values per head
    def _rows_key(self, cache: CacheHandle):
        return ("latent_rows", cache.kv.k.data_ptr())

    def _expands(self, ctx: StepContext, cache: CacheHandle) -> bool:
        """Whether this step takes the expanded road: bfloat16, not a decode step, every sequence at its
        first token (the step's tokens are all the keys), sizes the kernel and the products take, and,
        for a layer without a down projection, the rows the owning layer left in this step."""
        return (ctx.rt.dtype == torch.bfloat16 and not ctx.is_decode
                and ctx.total_kv_len == ctx.n_tokens and self.rank % 8 == 0 and self.row % 8 == 0
                and (self.n_heads * self.v_dim) % 8 == 0
                and ops.expanded_attention_supports(self.dim, self.rot, self.v_dim)
                and ((self.own_kv and cache.writes) or self._rows_key(cache) in ctx.shared))

    def _forward_expanded(self, x, ctx: StepContext, cache: CacheHandle, q, gate, dkv, rotation):
        rt = ctx.rt
        n, H = x.shape[0], self.n_heads
        if dkv is not None:
            rows = rt.empty(n, self.row, lifetime="step")
            ops.latent_prepare(q, dkv, rotation, self.norm_w, self.eps, cache.kv, ctx.token_seq, ctx.slots, ctx.positions,
                               None, H, self.dim, self.rot, self.rank, rows_out=rows, pairing=self.position.pairing)
            ctx.shared[self._rows_key(cache)] = rows
        else:
            rows = ctx.shared[self._rows_key(cache)]
            ops.latent_prepare(q, None, rotation, None, self.eps, None, ctx.token_seq, ctx.slots, ctx.positions,
                               None, H, self.dim, self.rot, self.rank, pairing=self.position.pairing)
        runs = rt.empty(n, H * (self.dim + self.v_dim + self.rot))
        ops.linear(rows[:, : self.rank], self.w_expand, runs)
        ops.latent_spread(rows[:, self.rank:], runs, H, self.dim + self.v_dim)
        heads = rt.empty(n, H * self.v_dim)
        ops.expanded_attention_bf16(q, runs, heads, ctx.cu_seqlens, ctx.n_seqs, ctx.max_q_len, H, self.dim, self.rot,
                                    self.v_dim, self.scale, self.window or 0, sinks=self.sinks)
        if gate is not None:
            ops.sigmoid_gate(heads, gate)
        return emit_update(heads, self.w_o, ctx)
