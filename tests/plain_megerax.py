"""Plain, slow Megerax decoder: the oracle of the numerics tests of that design.

Megerax is a decoder-only model whose config.json lists its layers one by one.
The embedded tokens pass an RMS norm; every layer is a pre-norm block around
one of three mixers and, where it has one, a gated feed-forward with the tanh
form of gelu; a final RMS norm, the head and a multiplier on the logits close
it.  The mixers:

* ``attention``: grouped-query attention with biased projections, a short
  causal convolution over time on every channel of q, k and v, a weighted RMS
  norm per query and key head, a rotation of interleaved pairs of the first
  channels of a head (frequencies scaled by wavelength), scores passed through
  c tanh(s / c), a sliding window, and an elementwise sigmoid gate on the
  concatenated heads.  A layer may read another layer's keys and values.
* ``latent_attention``: queries through a normed latent, keys and values
  through another normed latent plus one rotated key part that all heads
  share (half-split pairs), causal, and a learned number per head that joins
  the softmax's denominator without a key or a value.
* ``channel_delta``: the gated delta rule with a decay per head and key
  channel, S <- diag(g) S; S <- S + k (beta (v - S^T k))^T; o = S^T q, over
  convolved, silu-activated and unit-normed q and k, the read-out normed per
  head and gated through a low-rank sigmoid gate.

Whole sequences, no cache, one function per mechanism, NumPy in float64.  It
shares no code with the package.

Notation: W is stored [out, in]; rows of x are tokens, so a projection is x W^T.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def A(x):
    return np.asarray(x, F64)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = A(x)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * A(w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-A(z)))


def silu(z):
    z = A(z)
    return z * sigmoid(z)


def softplus(z):
    z = A(z)
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def gelu_tanh(z):
    z = A(z)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# --------------------------------------------------------------------------
# convolution over time
# --------------------------------------------------------------------------
def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j); the last
    column multiplies the current token, nothing stands before the start."""
    u, w = A(u), A(w)
    T, taps = u.shape[0], w.shape[1]
    y = np.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += u[: T - back] * w[:, j][None, :]
    return y


# --------------------------------------------------------------------------
# rotations
# --------------------------------------------------------------------------
def frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` (factor, low, high,
    original) a frequency whose wavelength is longer than original/low is
    divided by factor, one shorter than original/high stays, and those between
    are blended by s = (original/wavelength - low) / (high - low)."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return np.array(out, F64)


def rotate(x, positions, freqs, pairing):
    """x [T, heads, d]: the first 2 len(freqs) channels of every head turn,
    pair i by the angle position * freqs[i]; "interleaved" pairs channel 2i
    with 2i+1, "half" pairs i with i + len(freqs).  The rest pass."""
    x = np.array(x, F64)
    n = len(freqs)
    a = A(positions)[:, None] * freqs[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    if pairing == "interleaved":
        u, v = x[..., 0:2 * n:2].copy(), x[..., 1:2 * n:2].copy()
        x[..., 0:2 * n:2] = u * c - v * s
        x[..., 1:2 * n:2] = v * c + u * s
    elif pairing == "half":
        u, v = x[..., :n].copy(), x[..., n:2 * n].copy()
        x[..., :n] = u * c - v * s
        x[..., n:2 * n] = v * c + u * s
    else:
        raise ValueError(pairing)
    return x


# --------------------------------------------------------------------------
# softmax attention with the design's options
# --------------------------------------------------------------------------
def attend(q, k, v, scale, window=None, softcap=None, sinks=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Query i sees key j
    when 0 <= i - j (< window).  score = q . k * scale, then c tanh(score / c)
    with a cap c.  `sinks` [H]: exp(sink_h) joins head h's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen &= (i - j) < window
    out = np.zeros((T, H, v.shape[2]), F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = np.where(seen, s, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        if sinks is not None:
            m = np.maximum(m, float(sinks[h]))
        p = np.exp(s - m)
        den = p.sum(axis=-1, keepdims=True)
        if sinks is not None:
            den = den + np.exp(float(sinks[h]) - m)
        out[:, h] = (p / den) @ v[:, g]
    return out


def windowed_keys_values(h, w, m, eps):
    """What an attention layer with projections of its own caches: keys after
    convolution, norm and rotation [T, G, d], values after convolution [T, G, dv]."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ A(w["k"]).T + A(w["k.b"])
    v = h @ A(w["v"]).T + A(w["v.b"])
    if m.get("conv"):
        k, v = causal_conv(k, w["k.conv"]), causal_conv(v, w["v.conv"])
    k = rms_norm(k.reshape(T, G, d), w["k.norm"], eps)
    rot = m.get("rot")
    if rot:
        k = rotate(k, np.arange(T), frequencies(rot["dims"], rot["base"], rot.get("scaling")), "interleaved")
    return k, v.reshape(T, G, dv)


def attention_mixer(h, w, m, eps, kv=None):
    """The ``attention`` mixer.  `w`: the layer's tensors by short name; `m`: the
    mixer's block of config.json; `kv`: (keys, values) of the layer named by
    ``kv_from``, or None for a layer with projections of its own.  Returns
    (update, (keys, values))."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    if kv is None:
        kv = windowed_keys_values(h, w, m, eps)
    k, v = kv
    q = h @ A(w["q"]).T + A(w["q.b"])
    if m.get("conv"):
        q = causal_conv(q, w["q.conv"])
    q = rms_norm(q.reshape(T, H, d), w["q.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate(q, np.arange(T), frequencies(rot["dims"], rot["base"], rot.get("scaling")), "interleaved")
    a = attend(q, k, v, m["scale"], (m.get("mask") or {}).get("size"), m.get("softcap"))
    a = a.reshape(T, H * dv) * sigmoid(h @ A(w["g"]).T)
    return a @ A(w["o"]).T, kv


def latent_mixer(h, w, m, eps):
    """The ``latent_attention`` mixer."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    freqs = frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    pos = np.arange(T)
    cq = rms_norm(h @ A(w["dq"]).T, w["dq.norm"], eps)
    q = (cq @ A(w["uq"]).T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, freqs, "half")
    down = h @ A(w["dkv"]).T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate(down[:, None, rank:], pos, freqs, "half")                 # [T, 1, r], one for all heads
    k_plain = (c @ A(w["uk"]).T).reshape(T, H, d)
    v = (c @ A(w["uv"]).T).reshape(T, H, dv)
    qq = np.concatenate([q_plain, q_rot], axis=-1)
    kk = np.concatenate([k_plain, np.broadcast_to(k_rot, (T, H, r))], axis=-1)
    a = attend(qq, kk, v, m["scale"], (m.get("mask") or {}).get("size"), None, A(w["sink"]))
    return a.reshape(T, H * dv) @ A(w["o"]).T


# --------------------------------------------------------------------------
# the gated delta rule
# --------------------------------------------------------------------------
def unit_vector(x):
    x = A(x)
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """One head.  q, k, g [T, d]; v [T, dv]; beta [T].  S [d, dv] starts at zero;
    per token: S <- g[:, None] S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]), F64)
    out = np.zeros((T, v.shape[1]), F64)
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, w, m, eps):
    """The ``channel_delta`` mixer."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ A(w["q"]).T, h @ A(w["k"]).T, h @ A(w["v"]).T
    if m.get("conv"):
        q, k, v = causal_conv(q, w["q.conv"]), causal_conv(k, w["k.conv"]), causal_conv(v, w["v.conv"])
    q, k, v = silu(q), silu(k), silu(v)
    q = unit_vector(q.reshape(T, G, d)) * d ** -0.5
    k = unit_vector(k.reshape(T, G, d))
    v = v.reshape(T, H, dv)
    beta = sigmoid(h @ A(w["b"]).T)                                            # [T, H]
    step = softplus((h @ A(w["a1"]).T) @ A(w["a2"]).T + A(w["dt_bias"])).reshape(T, H, d)
    g = np.exp(-np.exp(A(w["A_log"]))[None, :, None] * step)                   # [T, H, d]
    o = np.zeros((T, H, dv), F64)
    for head in range(H):
        src = head // (H // G)
        o[:, head] = delta_rule(q[:, src], k[:, src], v[:, head], beta[:, head], g[:, head])
    gate = sigmoid((h @ A(w["g1"]).T) @ A(w["g2"]).T).reshape(T, H, dv)
    o = unit_rms(o, eps) * A(w["norm"]) * gate
    return o.reshape(T, H * dv) @ A(w["o"]).T


# --------------------------------------------------------------------------
# feed-forward, the whole model
# --------------------------------------------------------------------------
def gated_feed_forward(h, gate, up, down):
    return (gelu_tanh(h @ A(gate).T) * (h @ A(up).T)) @ A(down).T


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  `W`: every tensor by its full name;
    `layers_out`, a list, receives the hidden state after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = rms_norm(A(W["embed"])[np.asarray(tokens)], W["embed.norm"], eps)
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        w = {name[len(p) + 4:]: A(t) for name, t in W.items() if name.startswith(p + "mix.")}
        h = rms_norm(x, W[p + "norm1"], eps)
        kind = layer["type"]
        if kind == "attention":
            src = m.get("kv_from")
            update, kv = attention_mixer(h, w, m, eps, cached[src] if src is not None else None)
            cached[i] = kv
        elif kind == "latent_attention":
            update = latent_mixer(h, w, m, eps)
        elif kind == "channel_delta":
            update = delta_mixer(h, w, m, eps)
        else:
            raise ValueError(kind)
        x = x + update
        if layer.get("mlp") is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            x = x + gated_feed_forward(h, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"])
        if layers_out is not None:
            layers_out.append(x.copy())
    x = rms_norm(x, W["final.norm"], eps)
    return (x @ A(W["head"]).T) * float(cfg.get("logit_scale", 1.0))


def greedy(cfg, W, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, W, tokens)[-1])))
    return tokens[len(prompt):]
