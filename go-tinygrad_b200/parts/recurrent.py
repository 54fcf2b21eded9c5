"""Recurrent mixers: per-sequence state of fixed size instead of keys and values.

``mamba2``: the state-space mixer with a scalar decay per head.  With
inner = n_heads * head_dim, N = state_size, G = n_groups, the input projection
gives [z: inner | x: inner | B: G*N | C: G*N | dt: n_heads] per token.  x, B and
C pass a causal convolution over the last `conv_taps` tokens, per channel, and
silu.  Per head h (which reads B and C of group h // (n_heads / G)):

    dt_t = softplus(dt_t + dt_bias[h])
    S_t  = exp(-exp(a_log[h]) dt_t) S_{t-1} + dt_t B_t x_t^T        (S: N x head_dim)
    y_t  = S_t^T C_t + d[h] x_t

then y * silu(z), an RMS norm over `norm_parts` equal pieces of the row (each
piece by its own root mean square) with a weight, and the output projection.
What a sequence keeps between steps is S (float32) and the last
conv_taps - 1 inputs of the convolution; both live in the cache as
`StateRequest`s, are zero when a slot is opened, and are read and left by
every step, so a prompt, a portion of one and a single token are one code path.
Step sizes, decays, the state, the recurrence's sums and the norm are float32
in both compute dtypes, and so are B and C from the convolution on; the
projections and the x the convolution leaves are in the compute dtype.  The reference has no recurrent mixer.

Parameters: ``hidden_size``, ``n_heads``, ``head_dim``, ``state_size``,
``n_groups``, ``conv_taps``, ``norm_parts``, ``eps`` and the tensor names
``in``, ``conv``, ``conv_bias``, ``dt_bias``, ``a_log``, ``d``, ``norm``, ``o``.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..cache import CacheHandle, Request, StateRequest
from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Mixer, Runtime, StepContext, emit_update, register_part


@register_part("mixer", "mamba2")
class Mamba2(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.head_dim = int(self.param("head_dim"))
        self.n_state = int(self.param("state_size"))
        self.n_groups = int(self.param("n_groups"))
        self.taps = int(self.param("conv_taps"))
        self.norm_parts = int(self.p.get("norm_parts") or 1)
        self.eps = float(self.param("eps"))
        if self.n_heads % self.n_groups:
            raise ValueError(f"{self.n_heads} heads cannot share {self.n_groups} groups of B and C")
        self.inner = self.n_heads * self.head_dim
        if self.inner % self.norm_parts:
            raise ValueError(f"a row of {self.inner} cannot be normed in {self.norm_parts} equal pieces")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.conv_dim = self.inner + 2 * self.n_groups * self.n_state
        self.proj_dim = self.inner + self.conv_dim + self.n_heads
        self.names = {k: str(self.param(k)) for k in ("in", "conv", "conv_bias", "dt_bias", "a_log", "d", "norm", "o")}
        self.w_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        n = self.names
        return [WeightSpec(n["in"], (self.proj_dim, self.hidden)),
                WeightSpec(n["conv"], (self.conv_dim, self.taps), role="parameter", std=0.3),
                WeightSpec(n["conv_bias"], (self.conv_dim,), role="parameter", std=0.1),
                WeightSpec(n["dt_bias"], (self.n_heads,), role="parameter", mean=-1.5, std=0.7),
                WeightSpec(n["a_log"], (self.n_heads,), role="parameter", mean=-0.5, std=0.7),
                WeightSpec(n["d"], (self.n_heads,), role="parameter", mean=1.0, std=0.3),
                WeightSpec(n["norm"], (self.inner,), role="vector", mean=1.0),
                WeightSpec(n["o"], (self.hidden, self.inner))]

    def cache_requests(self) -> List[Request]:
        return [StateRequest("ssm", (self.n_heads, self.n_state, self.head_dim), "float32"),
                StateRequest("conv", (self.taps - 1, self.conv_dim), "float32")]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        n = self.names
        self.w_in = rt.matrix(tensors[n["in"]])
        self.w_o = rt.matrix(tensors[n["o"]])
        self.conv_w = rt.vector(tensors[n["conv"]].t().contiguous())      # tap by tap: [taps, channels]
        self.conv_b = rt.vector(tensors[n["conv_bias"]])
        self.dt_bias = rt.vector(tensors[n["dt_bias"]])
        self.a_log = rt.vector(tensors[n["a_log"]])
        self.d = rt.vector(tensors[n["d"]])
        self.norm_w = rt.vector(tensors[n["norm"]])

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        n = x.shape[0]
        if not cache.writes:
            raise ValueError("a recurrent mixer cannot read another run's state: every run advances its own")
        # rows padded to a multiple of 8 elements, which the products' stores want
        proj = rt.empty(n, (self.proj_dim + 7) // 8 * 8)[:, : self.proj_dim]
        ops.linear(x, self.w_in, proj)
        z = proj[:, : self.inner]
        conv_in = proj[:, self.inner: self.inner + self.conv_dim]
        dt_raw = proj[:, self.inner + self.conv_dim:]
        conv_state, ssm_state = cache.state("conv"), cache.state("ssm")
        # x in the compute dtype; B and C as float pairs, the form the recurrence reads
        xs = rt.empty(n, self.inner)
        bc = rt.empty(n, self.n_groups * self.n_state, 2, dtype=torch.float32)
        ops.causal_conv_silu(conv_in, self.conv_w, self.conv_b, conv_state, xs,
                             ctx.token_seq, ctx.cu_seqlens, ctx.slots, n_seqs=ctx.n_seqs, update_state=True,
                             one_token_each=ctx.is_decode, pairs=bc)
        ctx.trace("conv", xs)
        y = rt.empty(n, self.inner, dtype=torch.float32)
        ops.ssm_scan(xs, bc, dt_raw, self.dt_bias, self.a_log, self.d, ssm_state, y, ctx.cu_seqlens, ctx.slots,
                     ctx.n_seqs, self.n_heads, self.n_groups, self.n_state, self.head_dim,
                     one_token_each=ctx.is_decode)
        ctx.trace("scan", y)
        gated = rt.empty(n, self.inner)
        ops.gated_rmsnorm(y, z, self.norm_w, self.eps, gated, self.norm_parts)
        ctx.trace("attn", gated)
        return emit_update(gated, self.w_o, ctx)


@register_part("mixer", "gated_delta")
class GatedDelta(Mixer):
    """The gated delta rule with a decay per head and key channel.

    q = W_q x and k = W_k x (``n_kv_heads`` heads of ``head_dim``), v = W_v x
    (``n_heads`` heads of ``value_dim``; head h reads the queries and keys of
    group h // (n_heads / n_kv_heads)); each passes a causal convolution over
    the last ``conv_taps`` tokens per channel (no bias) and silu; q and k
    become unit vectors per head, x / sqrt(sum(x^2) + ``unit_eps``), q also times
    head_dim^-1/2.  beta = sigmoid(W_b x), one per head; the decay
    g = exp(-exp(a_log[h]) softplus(W_a2 (W_a1 x) + dt_bias)), one per head and
    key channel.  Per head, token by token,

        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

    (S: head_dim x value_dim, zero at the start).  Every head of o is divided by
    its root mean square (``eps``), multiplied by a weight of value_dim channels
    that the heads share and by sigmoid(W_g2 (W_g1 x)), and projected by W_o.
    What a sequence keeps between steps is S and the last conv_taps - 1 inputs of
    the convolution, both float32 `StateRequest`s.  Unit norms, beta, the decay
    with its softplus and exponentials, the state, the sums of the recurrence and
    the norm of the read-out are float32 in both compute dtypes; the projections
    leave float32 sums that the convolution reads.  The widths of the two
    low-rank projections are those of their tensors unless ``decay_rank`` and
    ``gate_rank`` name them.  The reference has no recurrent mixer.

    Parameters: ``hidden_size``, ``n_heads``, ``n_kv_heads``, ``head_dim``,
    ``value_dim``, ``conv_taps`` (None: no convolution), ``eps``, ``unit_eps``,
    ``decay_rank``, ``gate_rank`` and the tensor names ``q``, ``k``, ``v``,
    ``q_conv``, ``k_conv``, ``v_conv``, ``beta``, ``a_log``, ``decay_down``,
    ``decay_up``, ``dt_bias``, ``gate_down``, ``gate_up``, ``norm``, ``o``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.n_kv = int(self.param("n_kv_heads"))
        self.dim = int(self.param("head_dim"))
        self.vdim = int(self.param("value_dim"))
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} heads cannot share {self.n_kv} heads of queries and keys")
        taps = self.p.get("conv_taps")
        self.taps = int(taps) if taps else 1
        self.eps = float(self.param("eps"))
        self.unit_eps = float(self.p.get("unit_eps") or 1e-6)
        self.decay_rank = int(self.p.get("decay_rank") or -1)
        self.gate_rank = int(self.p.get("gate_rank") or -1)
        if self.dim > ops.DELTA_MAX_KEY_DIM:
            raise ValueError(f"heads of {self.dim} key channels are more than the recurrence's kernel takes "
                             f"({ops.DELTA_MAX_KEY_DIM})")
        wanted = ["q", "k", "v", "beta", "a_log", "decay_down", "decay_up", "dt_bias", "gate_down", "gate_up", "norm", "o"]
        if self.taps > 1:
            wanted += ["q_conv", "k_conv", "v_conv"]
        self.names = {k: str(self.param(k)) for k in wanted}
        self.qk_width = 2 * self.n_kv * self.dim
        self.v_width = self.n_heads * self.vdim
        self.conv_dim = self.qk_width + self.v_width
        self.g_width = self.n_heads * self.dim

    def weight_specs(self) -> List[WeightSpec]:
        n, low = self.names, max(8, self.dim // 4)
        specs = [WeightSpec(n["q"], (self.n_kv * self.dim, self.hidden)),
                 WeightSpec(n["k"], (self.n_kv * self.dim, self.hidden)),
                 WeightSpec(n["v"], (self.v_width, self.hidden)),
                 WeightSpec(n["beta"], (self.n_heads, self.hidden)),
                 WeightSpec(n["a_log"], (self.n_heads,), role="parameter", mean=-0.5, std=0.7),
                 WeightSpec(n["decay_down"], (self.decay_rank, self.hidden), free_size=low),
                 WeightSpec(n["decay_up"], (self.g_width, self.decay_rank), free_size=low, std=0.1),
                 WeightSpec(n["dt_bias"], (self.g_width,), role="parameter", mean=-1.5, std=0.7),
                 WeightSpec(n["gate_down"], (self.gate_rank, self.hidden), free_size=low),
                 WeightSpec(n["gate_up"], (self.v_width, self.gate_rank), free_size=low, std=0.1),
                 WeightSpec(n["norm"], (self.vdim,), role="vector", mean=1.0),
                 WeightSpec(n["o"], (self.hidden, self.v_width))]
        if self.taps > 1:
            specs += [WeightSpec(n[k], (size, self.taps), role="parameter", mean=1.0 / self.taps, std=0.3)
                      for k, size in (("q_conv", self.n_kv * self.dim), ("k_conv", self.n_kv * self.dim), ("v_conv", self.v_width))]
        return specs

    def cache_requests(self) -> List[Request]:
        requests: List[Request] = [StateRequest("delta", (self.n_heads, self.dim, self.vdim), "float32")]
        if self.taps > 1:
            requests.append(StateRequest("conv", (self.taps - 1, self.conv_dim), "float32"))
        return requests

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        n = self.names
        decay_down, decay_up = tensors[n["decay_down"]], tensors[n["decay_up"]]
        gate_down, gate_up = tensors[n["gate_down"]], tensors[n["gate_up"]]
        if decay_down.shape[0] != decay_up.shape[1] or gate_down.shape[0] != gate_up.shape[1]:
            raise ValueError(f"the two halves of a low-rank projection disagree: {n['decay_down']} {list(decay_down.shape)} and "
                             f"{n['decay_up']} {list(decay_up.shape)}, {n['gate_down']} {list(gate_down.shape)} and "
                             f"{n['gate_up']} {list(gate_up.shape)}")
        self.r_decay, self.r_gate = int(decay_down.shape[0]), int(gate_down.shape[0])
        # two products read x: [q | k | v | beta], which leaves float sums, and the narrow halves of the low-rank
        # projections [decay_down | gate_down], in the compute dtype as operands of the products that widen them;
        # rows padded to a multiple of 8
        def stacked(keys):
            parts = [tensors[n[k]].to(rt.dtype) for k in keys]
            rows = sum(p.shape[0] for p in parts)
            if rows % 8:
                parts.append(torch.zeros((8 - rows % 8, self.hidden), dtype=rt.dtype, device=parts[0].device))
            return rt.matrix(torch.cat(parts, dim=0))
        self.w_in = stacked(("q", "k", "v", "beta"))
        self.w_low = stacked(("decay_down", "gate_down"))
        self.w_decay_up = rt.matrix(decay_up)
        self.w_gate_up = rt.matrix(gate_up)
        self.w_o = rt.matrix(tensors[n["o"]])
        self.a_log = rt.vector(tensors[n["a_log"]])
        self.dt_bias = rt.vector(tensors[n["dt_bias"]].reshape(-1))
        self.norm_w = rt.vector(tensors[n["norm"]])
        self.conv_w = None
        if self.taps > 1:
            self.conv_w = rt.vector(torch.cat([tensors[n[k]].to(torch.float32) for k in ("q_conv", "k_conv", "v_conv")],
                                              dim=0).t().contiguous())      # tap by tap: [taps, channels]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        n = x.shape[0]
        if not cache.writes:
            raise ValueError("a recurrent mixer cannot read another run's state: every run advances its own")
        sums = rt.empty(n, self.w_in.shape[0], dtype=torch.float32)
        ops.linear(x, self.w_in, sums)
        beta_in = sums[:, self.conv_dim: self.conv_dim + self.n_heads]
        narrow = rt.empty(n, self.w_low.shape[0])
        ops.linear(x, self.w_low, narrow)
        if self.taps > 1:
            qkv = rt.empty(n, self.conv_dim, dtype=torch.float32)
            ops.causal_conv_silu(sums[:, : self.conv_dim], self.conv_w, None, cache.state("conv"), qkv, ctx.token_seq,
                                 ctx.cu_seqlens, ctx.slots, n_seqs=ctx.n_seqs, update_state=True,
                                 one_token_each=ctx.is_decode)
        else:
            qkv = sums[:, : self.conv_dim]
            ops.activation(qkv, "silu")
        ctx.trace("conv", qkv)
        decay = rt.empty(n, self.g_width, dtype=torch.float32)
        ops.linear(narrow[:, : self.r_decay], self.w_decay_up, decay)
        gate = rt.empty(n, self.v_width, dtype=torch.float32)
        ops.linear(narrow[:, self.r_decay: self.r_decay + self.r_gate], self.w_gate_up, gate)
        beta = rt.empty(n, self.n_heads, dtype=torch.float32)
        ops.delta_prepare(qkv, decay, self.dt_bias, self.a_log, beta_in, beta, self.n_heads, self.n_kv, self.dim,
                          self.unit_eps, self.dim ** -0.5)
        y = rt.empty(n, self.v_width, dtype=torch.float32)
        ops.delta_scan(qkv, qkv[:, self.qk_width:], decay, beta, cache.state("delta"), y, ctx.cu_seqlens, ctx.slots,
                       ctx.n_seqs, self.n_heads, self.n_kv, self.dim, self.vdim, one_token_each=ctx.is_decode)
        ctx.trace("scan", y)
        out = rt.empty(n, (self.v_width + 7) // 8 * 8)[:, : self.v_width]
        ops.head_norm_gate(y, gate, self.norm_w, self.eps, out, self.n_heads)
        ctx.trace("attn", out)
        return emit_update(out, self.w_o, ctx)
