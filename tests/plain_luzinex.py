"""A plain, slow implementation of the Luzinex decoder in NumPy float64: whole sequences, no
cache, no batching, one function per mechanism.  It shares no code with the engine and is the
oracle its kernels are compared with.

Notation.  ``W`` of a linear map is stored ``[out, in]`` and applied as ``x @ W.T``.  A sequence
is ``T`` tokens at positions ``0 .. T-1``.  A layer is ``x + mixer(n1(x)) + ff(n2(x))``: both
branches read the same ``x``.

* ``rms_norm``            ``x / sqrt(mean(x^2) + eps) * w``
* ``rotate_half`` / ``rotate_pairs``   rotary positions over the first ``dims`` channels of a head, channel
                          ``i`` paired with ``i + dims/2`` or channel ``2i`` with ``2i + 1``
* ``gelu_ff``             ``W_d (gelu_tanh(W_g x) * (W_u x))``
* ``latent_attention``    queries through a normed latent, keys and values expanded from a normed latent that is
                          shared by all heads, one rotated key part shared by all heads, gated output
* ``sink_window_attention``   keys are also the values, sliding window that keeps the first tokens, a learned
                          term in the softmax denominator, gated output
* ``retention``           linear attention with a fixed decay per head, read-out normalised per head, gated
"""
from __future__ import annotations

import numpy as np

ROUND = None          # a function applied to activations where a bfloat16 engine rounds; None = exact


def _r(x):
    return x if ROUND is None else ROUND(x)


def round_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint32) << 16
    return u.view(np.float32).astype(np.float64)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


# ----------------------------------------------------------------------------- norm

def rms_norm(x, w, eps):
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


# ----------------------------------------------------------------------------- rotary positions

def _angles(positions, dims, base):
    i = np.arange(dims // 2, dtype=np.float64)
    return np.asarray(positions, dtype=np.float64)[:, None] * np.power(float(base), -2.0 * i / dims)[None, :]


def rotate_half(x, positions, dims, base):
    """x [T, heads, d]: channel i with channel i + dims/2, i < dims/2; the rest unchanged."""
    a = _angles(positions, dims, base)[:, None, :]
    c, s = np.cos(a), np.sin(a)
    out = np.array(x, dtype=np.float64, copy=True)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out[..., :dims // 2] = u * c - v * s
    out[..., dims // 2:dims] = v * c + u * s
    return out


def rotate_pairs(x, positions, dims, base):
    """x [T, heads, d]: channel 2i with channel 2i + 1, i < dims/2; the rest unchanged."""
    a = _angles(positions, dims, base)[:, None, :]
    c, s = np.cos(a), np.sin(a)
    out = np.array(x, dtype=np.float64, copy=True)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- feed-forward

def gelu_ff(x, w_gate, w_up, w_down):
    g, u = _r(x @ w_gate.T), _r(x @ w_up.T)
    return _r(_r(gelu_tanh(g) * u) @ w_down.T)


# ----------------------------------------------------------------------------- softmax attention

def visible(T, window=0, keep_first=0):
    """[T, T] bool: query i sees key j."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    m = j <= i
    if window > 0:
        m &= (i - j < window) | (j < keep_first)
    return m


def masked_softmax(scores, mask, sink=None):
    """scores [H, T, T]; sink [H] adds exp(sink_h) to every denominator of head h."""
    s = np.where(mask[None], scores, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink[:, None, None])
    e = np.exp(s - m)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None, None] - m)
    return e / den


def latent_keys(h, w_dkv, norm_w, eps, kv_rank, rot_dim, base, positions):
    """What a latent layer keeps per token: the normed latent [T, kv_rank] and the rotated shared key part."""
    d = _r(h @ w_dkv.T)
    c = _r(rms_norm(d[:, :kv_rank], norm_w, eps))
    kr = _r(rotate_half(d[:, None, kv_rank:kv_rank + rot_dim], positions, rot_dim, base)[:, 0])
    return c, kr


def latent_attention(h, p, m, eps, kept=None):
    """p: tensors by short name (dq, dq.norm, uq, [dkv, dkv.norm,] uk, uv, g, o); m: the mixer's sizes.
    ``kept``: (latent, rotated key part) of the layer whose keys this one reads instead of making its own.
    Returns (delta, kept)."""
    T = h.shape[0]
    H, dim, rot, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    cq = _r(rms_norm(_r(h @ p["dq"].T), p["dq.norm"], eps))
    q = _r(cq @ p["uq"].T).reshape(T, H, dim + rot)
    qn, qr = q[..., :dim], _r(rotate_half(q[..., dim:], pos, rot, m["rot"]["base"]))
    if kept is None:
        kept = latent_keys(h, p["dkv"], p["dkv.norm"], eps, rank, rot, m["rot"]["base"], pos)
    c, kr = kept
    kn = _r(c @ p["uk"].T).reshape(T, H, dim)
    v = _r(c @ p["uv"].T).reshape(T, H, vd)
    s = (np.einsum("ihd,jhd->hij", qn, kn) + np.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    w = masked_softmax(s, visible(T))
    o = _r(np.einsum("hij,jhd->ihd", w, v).reshape(T, H * vd))
    o = _r(o * sigmoid(_r(h @ p["g"].T)))
    return _r(o @ p["o"].T), kept


def sink_window_attention(h, p, m):
    """p: q, k, sink, g, o."""
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = _r(h @ p["q"].T).reshape(T, H, dim)
    k = _r(h @ p["k"].T).reshape(T, G, dim)
    v = k[..., :vd]
    q = _r(rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"]))
    k = _r(rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"]))
    rep = H // G
    ke, ve = np.repeat(k, rep, axis=1), np.repeat(v, rep, axis=1)
    s = np.einsum("ihd,jhd->hij", q, ke) * m["scale"]
    mask = m.get("mask") or {}
    w = masked_softmax(s, visible(T, int(mask.get("size", 0)), int(mask.get("keep_first", 0))), p["sink"])
    o = _r(np.einsum("hij,jhd->ihd", w, ve).reshape(T, H * vd))
    o = _r(o * sigmoid(_r(h @ p["g"].T)))
    return _r(o @ p["o"].T)


# ----------------------------------------------------------------------------- retention

def retention(h, p, m, eps, state=None):
    """p: q, k, v, g, o.  Token after token: S <- decay_h S + k v^T, o = S^T q.  Returns (delta, state)."""
    T = h.shape[0]
    H, dim, vd = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    q = _r(rotate_half(_r(h @ p["q"].T).reshape(T, H, dim), pos, m["rot"]["dims"], m["rot"]["base"]))
    k = _r(rotate_half(_r(h @ p["k"].T).reshape(T, H, dim), pos, m["rot"]["dims"], m["rot"]["base"]))
    k = k * dim ** -0.5
    v = _r(h @ p["v"].T).reshape(T, H, vd)
    S = np.zeros((H, dim, vd)) if state is None else np.array(state, dtype=np.float64)
    decay = np.asarray(m["decay"], dtype=np.float64)
    o = np.zeros((T, H, vd))
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, None, eps).reshape(T, H * vd)
    o = _r(o * silu(_r(h @ p["g"].T)))
    return _r(o @ p["o"].T), S


# ----------------------------------------------------------------------------- the model

def _layer_tensors(weights, i, part):
    pre = f"l{i}.{part}."
    return {k[len(pre):]: v for k, v in weights.items() if k.startswith(pre)}


def forward(config, weights, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out`` (a list) receives the residual stream
    after every layer."""
    eps = config["norm"]["eps"]
    x = np.asarray(weights["embed"], dtype=np.float64)[np.asarray(tokens)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        p = _layer_tensors(weights, i, "mix")
        h = _r(rms_norm(x, weights[f"l{i}.norm1"], eps))
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            d, kept[i] = latent_attention(h, p, m, eps, kept[src] if src is not None else None)
        elif layer["type"] == "attention":
            d = sink_window_attention(h, p, m)
        elif layer["type"] == "retention":
            d, _ = retention(h, p, m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            f = _layer_tensors(weights, i, "mlp")
            d = d + gelu_ff(_r(rms_norm(x, weights[f"l{i}.norm2"], eps)), f["gate"], f["up"], f["down"])
        x = x + d
        if layers_out is not None:
            layers_out.append(x.copy())
    hn = _r(rms_norm(x, weights["final.norm"], eps))
    return hn @ np.asarray(weights["head"], dtype=np.float64).T
