"""Plain, slow Zotolix decoder: the oracle of the numerics tests of that design.

Zotolix is a decoder-only model whose config.json lists its layers one by one.
The hidden state is kept in several copies (hyper-connections): a sublayer
reads a weighted sum of the copies through an RMS norm, and its output goes
back into every copy with a weight of its own while the copies are remixed by a
small matrix.  Mixers are grouped-query attention over keys of the query's own
chunk of positions, with biased projections, a rotation of the first channels
of a head, values blended with the values of the first blending layer, and
either unit-norm queries and keys (``attention``) or a sigmoid gate per head
(``attention_2``).  The feed-forward is a mixture of squared-relu experts whose
sigmoid router score scales the expert's input.

Whole sequences, no cache, one function per mechanism, NumPy in float64.  It
shares no code with the package.

Notation: W is stored [out, in]; rows of x are tokens, so a projection is x W^T.
"""
from __future__ import annotations

import numpy as np

F64 = np.float64


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, F64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * np.asarray(w, F64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F64)))


# --------------------------------------------------------------------------
# rotation of the first `dims` channels of a head, pairs (i, i + dims/2)
# --------------------------------------------------------------------------
def rotate_heads(x, positions, dims, base):
    """x [T, heads, d]; channel i < dims/2 and channel i + dims/2 turn by the
    angle position * base^(-2i/dims); channels from `dims` on pass."""
    x = np.array(x, F64)
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], F64)
    a = np.asarray(positions, F64)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half].copy(), x[..., half:dims].copy()
    x[..., :half] = u * c - v * s
    x[..., half:dims] = v * c + u * s
    return x


# --------------------------------------------------------------------------
# attention over the query's own chunk
# --------------------------------------------------------------------------
def chunk_visible(i, j, size):
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    return size is None or i // size == j // size


def attend(q, k, v, scale, size):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]: softmax over the
    visible keys of (q . k) scale; query head h reads key/value head h // (H/G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (j <= i) if size is None else (j <= i) & (i // size == j // size)     # chunk_visible, all pairs
    out = np.zeros((T, H, v.shape[2]), F64)
    for h in range(H):
        g = h // (H // G)
        s = np.where(seen, (q[:, h] @ k[:, g].T) * scale, -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, h] = (p / p.sum(axis=-1, keepdims=True)) @ v[:, g]
    return out


def blend_values(v, v_first, lam):
    """(1 - lam) v + lam v_first."""
    return (1.0 - lam) * np.asarray(v, F64) + lam * np.asarray(v_first, F64)


def attention_mixer(h, w, p, layer_type, eps, v_first=None):
    """One mixer.  `w`: the layer's tensors by short name (q, q.b, k, k.b, v,
    v.b, vmix, g, o); `p`: heads, kv_heads, dim, vdim, rot_dims, rot_base, scale,
    mask_size.  `v_first`: the first blending layer's values [T, G, dv], or None
    when this layer does not blend (or is that first layer).  Returns (update,
    the values this layer caches)."""
    T = h.shape[0]
    H, G, d, dv = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = (h @ np.asarray(w["q"], F64).T + w["q.b"]).reshape(T, H, d)
    k = (h @ np.asarray(w["k"], F64).T + w["k.b"]).reshape(T, G, d)
    v = (h @ np.asarray(w["v"], F64).T + w["v.b"]).reshape(T, G, dv)
    pos = np.arange(T)
    q = rotate_heads(q, pos, p["rot_dims"], p["rot_base"])
    k = rotate_heads(k, pos, p["rot_dims"], p["rot_base"])
    if layer_type == "attention":
        q, k = unit_rms(q, eps), unit_rms(k, eps)
    if v_first is not None:
        v = blend_values(v, v_first, float(w["vmix"]))
    a = attend(q, k, v, p["scale"], p["mask_size"])
    if layer_type == "attention_2":
        a = a * sigmoid(h @ np.asarray(w["g"], F64).T)[:, :, None]
    return a.reshape(T, H * dv) @ np.asarray(w["o"], F64).T, v


# --------------------------------------------------------------------------
# mixture of squared-relu experts; the router's score scales the input
# --------------------------------------------------------------------------
def choose_experts(h, router, top):
    """(indices [T, top], scores [T, top]): the `top` largest sigmoid scores, a
    tie going to the lower index; the scores are the weights as they are."""
    s = sigmoid(h @ np.asarray(router, F64).T)
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1)


def expert(x, up, down):
    z = np.maximum(x @ np.asarray(up, F64).T, 0.0)
    return (z * z) @ np.asarray(down, F64).T


def mixture(h, router, ups, downs, top, chosen=None):
    """sum over a token's experts of expert(score * h).  `chosen` [T, top]
    overrides the choice (the scores stay the router's own)."""
    s = sigmoid(h @ np.asarray(router, F64).T)
    idx = choose_experts(h, router, top)[0] if chosen is None else np.asarray(chosen)
    out = np.zeros((h.shape[0], np.asarray(downs[0]).shape[0]), F64)
    for t in range(h.shape[0]):
        for e in idx[t]:
            out[t] += expert(s[t, e] * h[t], ups[e], downs[e])
    return out


# --------------------------------------------------------------------------
# hyper-connections
# --------------------------------------------------------------------------
def streams_read(xs, w_in):
    """xs [S, T, W] -> sum_s in[s] xs[s]."""
    return np.tensordot(np.asarray(w_in, F64), xs, axes=(0, 0))


def streams_write(xs, y, mix, w_out, m):
    """new[t] = sum_s mix[s, t] xs[s] + m out[t] y, all copies at once."""
    new = np.tensordot(np.asarray(mix, F64).T, xs, axes=(1, 0))
    return new + m * np.asarray(w_out, F64)[:, None, None] * y[None]


# --------------------------------------------------------------------------
# the whole model
# --------------------------------------------------------------------------
def _mixer_params(m):
    return {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
            "rot_dims": m["rot"]["dims"], "rot_base": m["rot"]["base"], "scale": m["scale"],
            "mask_size": (m.get("mask") or {}).get("size")}


def forward(cfg, W, tokens, experts_of=None, layers_out=None):
    """Logits [T, vocab] of one sequence.  `W`: every tensor by its full name.
    `experts_of[(layer)]` [T, top] overrides a layer's expert choice;
    `layers_out`, a list, receives the hidden state (the sum of the copies)
    after every layer."""
    eps = cfg["norm"]["eps"]
    m = float(cfg.get("residual_mult", 1.0))
    S = cfg.get("streams")
    x0 = np.asarray(W["embed"], F64)[np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    xs = np.stack([x0] * (S or 1))
    v_first = None

    def sub(xs, li, q, fn):
        p = f"l{li}."
        if S:
            u = streams_read(xs, W[p + f"hc{q}.in"])
        else:
            u = xs[0]
        y = fn(rms_norm(u, W[p + f"norm{q}"], eps))
        if S:
            return streams_write(xs, y, W[p + f"hc{q}.mix"], W[p + f"hc{q}.out"], m)
        return xs + m * y[None]

    for li, layer in enumerate(cfg["layers"]):
        p = f"l{li}."
        mp = _mixer_params(layer["mixer"])
        blends = bool(layer["mixer"].get("v_mix"))
        w = {k[len(p) + 4:]: np.asarray(v, F64) for k, v in W.items() if k.startswith(p + "mix.")}
        kept = {}

        def mixer(h):
            upd, v = attention_mixer(h, w, mp, layer["type"], eps, v_first if blends else None)
            kept["v"] = v
            return upd
        xs = sub(xs, li, 1, mixer)
        if blends and v_first is None:
            v_first = kept["v"]
        mlp = layer.get("mlp")
        if mlp is not None:
            E, top = mlp["router"]["experts"], mlp["router"]["top"]
            ups = [W[p + f"mlp.e{e}.up"] for e in range(E)]
            downs = [W[p + f"mlp.e{e}.down"] for e in range(E)]
            chosen = None if experts_of is None else experts_of.get(li)
            xs = sub(xs, li, 2, lambda h: mixture(h, W[p + "mlp.router"], ups, downs, top, chosen))
        if layers_out is not None:
            layers_out.append(xs.sum(axis=0))
    x = xs.sum(axis=0)
    return rms_norm(x, W["final.norm"], eps) @ np.asarray(W["embed"], F64).T


def greedy(cfg, W, prompt, n_new):
    """n_new tokens, each the first maximum of the logits after everything before it."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(np.argmax(forward(cfg, W, seq)[-1])))
    return seq[len(prompt):]
