"""A plain, slow implementation of the Notirax decoder in NumPy float64: whole
sequences, no cache, no batching, one function per mechanism.  It shares no code
with the engine and is the oracle its kernels are compared with.

Notation.  ``W`` of a linear map is stored ``[out, in]`` and applied as ``x @ W.T``.
A sequence is ``T`` tokens at positions ``0 .. T-1``.

* ``sinusoid``        position vector: pair ``i`` holds ``sin(p f_i), cos(p f_i)``, ``f_i = 10000^(-2i/width)``
* ``group_rms_norm``  the vector cut into equal consecutive groups, each scaled by its own root mean square
* ``hyper_read`` / ``hyper_write``   several residual streams: a weighted read-in, a mixing matrix and a write-out
* ``talking_chunk_attention``  biased projections, soft-capped scores mixed across heads, chunk-local causal mask
* ``channel_delta``   gated delta rule with one decay per head and key channel, short convolutions before it
* ``grouped_router`` / ``clamped_expert`` / ``moe``   sigmoid router limited to the best groups, clamped gated experts
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


def softplus(x):
    return np.logaddexp(0.0, x)


def silu(x):
    return x * sigmoid(x)


# ----------------------------------------------------------------------------- embedding

def sinusoid(positions, width):
    p = np.asarray(positions, dtype=np.float64)[:, None]
    i = np.arange((width + 1) // 2, dtype=np.float64)[None, :]
    ang = p * np.power(10000.0, -2.0 * i / width)
    out = np.zeros((p.shape[0], 2 * ((width + 1) // 2)))
    out[:, 0::2] = np.sin(ang)
    out[:, 1::2] = np.cos(ang)
    return out[:, :width]


def embed(table, tokens, positions):
    return table[np.asarray(tokens)] + sinusoid(positions, table.shape[1])


# ----------------------------------------------------------------------------- norm

def group_rms_norm(x, w, eps, groups):
    T, H = x.shape
    g = x.reshape(T, groups, H // groups)
    g = g / np.sqrt(np.mean(g * g, axis=-1, keepdims=True) + eps)
    return g.reshape(T, H) * w


# ----------------------------------------------------------------------------- residual streams

def hyper_read(streams, w_in):
    """streams [S, T, H] -> sum_s in[s] * streams[s]."""
    return np.einsum("s,sth->th", w_in, streams)


def hyper_write(streams, y, w_mix, w_out):
    """new[t] = sum_s mix[s, t] * old[s] + out[t] * y, all streams at once from the old ones."""
    return np.einsum("sr,sth->rth", w_mix, streams) + w_out[:, None, None] * y[None]


# ----------------------------------------------------------------------------- attention

def talking_chunk_attention(h, p, W):
    """``p``: the mixer's sizes and constants; ``W(name)``: the mixer's tensor or None."""
    T = h.shape[0]
    nh, nkv, d, dv = p["heads"], p["kv_heads"], p["dim"], p["vdim"]

    def lin(name, x):
        y = x @ W(name).T
        b = W(name + ".b")
        return y if b is None else y + b

    q = _r(lin("q", h)).reshape(T, nh, d)
    k = _r(lin("k", h)).reshape(T, nkv, d)
    v = _r(lin("v", h)).reshape(T, nkv, dv)
    rep = nh // nkv
    s = np.empty((nh, T, T))
    for a in range(nh):
        s[a] = q[:, a] @ k[:, a // rep].T
    s = s * p["scale"]
    cap = p.get("softcap")
    if cap:
        s = cap * np.tanh(s / cap)
    talk = W("talk")
    if talk is not None:
        s = np.einsum("hg,gij->hij", talk, s)
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    seen = j <= i
    size = (p.get("mask") or {}).get("size")
    if size:
        seen = seen & (i // size == j // size)
    s = np.where(seen[None], s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    pr = e / e.sum(axis=-1, keepdims=True)
    o = np.empty((T, nh, dv))
    for a in range(nh):
        o[:, a] = pr[a] @ v[:, a // rep]
    return lin("o", _r(o.reshape(T, nh * dv)))


# ----------------------------------------------------------------------------- gated delta rule

def short_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]: y[t, c] = sum_j w[c, j] x[t - (taps-1) + j, c], zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += pad[j:j + T] * taps_w[:, j][None, :]
    return y


def channel_delta(h, p, W, eps):
    T = h.shape[0]
    nh, nkv, d, dv = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    rep = nh // nkv
    q = _r(silu(short_conv(_r(h @ W("q").T), W("q.conv")))).reshape(T, nkv, d)
    k = _r(silu(short_conv(_r(h @ W("k").T), W("k.conv")))).reshape(T, nkv, d)
    v = _r(silu(short_conv(_r(h @ W("v").T), W("v.conv")))).reshape(T, nh, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W("b").T)                                              # [T, nh]
    dt = softplus(_r(h @ W("a1").T) @ W("a2").T + W("dt_bias")).reshape(T, nh, d)
    decay = np.exp(-np.exp(W("A_log"))[None, :, None] * dt)                   # [T, nh, d]
    o = np.empty((T, nh, dv))
    for a in range(nh):
        S = np.zeros((d, dv))
        for t in range(T):
            kt, qt = k[t, a // rep], q[t, a // rep]
            S = decay[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ kt)
            S = S + np.outer(kt, u)
            o[t, a] = S.T @ qt
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps) * W("norm")
    gate = sigmoid(_r(h @ W("g1").T) @ W("g2").T).reshape(T, nh, dv)
    return _r((o * gate).reshape(T, nh * dv)) @ W("o").T


# ----------------------------------------------------------------------------- mixture of experts

def grouped_router(h, w_router, r):
    """-> (chosen experts [T, top], their weights [T, top])."""
    s = sigmoid(h @ w_router.T)
    T, E = s.shape
    allowed = np.ones((T, E), dtype=bool)
    g = r.get("groups")
    if g:
        per = E // g["count"]
        sg = s.reshape(T, g["count"], per)
        best2 = np.sort(sg, axis=-1)[:, :, -2:].sum(axis=-1)
        keep = np.argsort(-best2, axis=-1, kind="stable")[:, :g["keep"]]
        ok = np.zeros((T, g["count"]), dtype=bool)
        np.put_along_axis(ok, keep, True, axis=-1)
        allowed = np.repeat(ok, per, axis=-1)
    masked = np.where(allowed, s, -np.inf)
    chosen = np.argsort(-masked, axis=-1, kind="stable")[:, :r["top"]]
    return chosen, np.take_along_axis(s, chosen, axis=-1) * r.get("scale", 1.0)


def clamped_expert(h, w_gate, w_up, w_down, limit):
    g = np.minimum(h @ w_gate.T, limit)
    u = np.clip(h @ w_up.T, -limit, limit)
    return _r(g * sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def moe(h, p, W):
    chosen, weight = grouped_router(h, W("router"), p["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weight[t]):
            out[t] += wt * clamped_expert(h[t:t + 1], W(f"e{e}.gate"), W(f"e{e}.up"), W(f"e{e}.down"),
                                          p["expert"]["limit"])[0]
    return out


# ----------------------------------------------------------------------------- the model

def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  ``w``: name -> float64 array.  ``layers_out``: a list that
    receives the residual stream (the sum of the streams) after every layer."""
    T = len(tokens)
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x0 = embed(w["embed"], tokens, np.arange(T))
    S = cfg.get("streams")
    streams = np.repeat(x0[None], S or 1, axis=0)
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        subs = [("mix.", "norm1", "hc1.", layer["type"], layer["mixer"])]
        if layer.get("mlp") is not None:
            subs.append(("mlp.", "norm2", "hc2.", layer["mlp"]["kind"], layer["mlp"]))
        for sub, norm, hc, kind, p in subs:
            W = lambda name, _p=pre + sub: w.get(_p + name)
            u = hyper_read(streams, w[pre + hc + "in"]) if S else streams[0]
            hn = _r(group_rms_norm(u, w[pre + norm], eps, groups))
            if kind == "attention":
                y = talking_chunk_attention(hn, p, W)
            elif kind == "channel_delta":
                y = channel_delta(hn, p, W, eps)
            elif kind == "moe":
                y = moe(hn, p, W)
            else:
                raise ValueError(kind)
            y = _r(y)
            streams = hyper_write(streams, y, w[pre + hc + "mix"], w[pre + hc + "out"]) if S else streams + y[None]
        if layers_out is not None:
            layers_out.append(streams.sum(axis=0))
    x = streams.sum(axis=0)
    return _r(group_rms_norm(x, w["final.norm"], eps, groups)) @ w["embed"].T


def generate(cfg, w, prompt, n):
    seq = list(prompt)
    out = []
    for _ in range(n):
        t = int(np.argmax(forward(cfg, w, seq)[-1]))
        out.append(t)
        seq.append(t)
    return out
