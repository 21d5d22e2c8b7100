"""Small Notirax configurations that differ in every size and option, random weights for them
(made here, not by the engine's random-weights mode) and model folders written by the tests' own
writer."""
from __future__ import annotations

import numpy as np

from helpers import bf16_round, write_model_dir


def _attn(heads, kv, dim, vdim, chunk, softcap, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "softcap": softcap,
         "scale": dim ** -0.5 if scale is None else scale}
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m}


def _delta(heads, kv, dim, vdim, conv):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _moe(ff, experts, top, groups=None, keep=None, scale=1.0, limit=2.0):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# odd sizes everywhere: key and value sizes differ, grouped keys in the delta rule, a chunk that is no
# multiple of the page, a layer without a feed-forward, two streams, three norm groups
NX_A = {"architecture": "Notirax", "vocab": 101, "width": 48, "streams": 2, "norm": {"eps": 1e-5, "groups": 3},
        "layers": [_layer(_delta(4, 2, 8, 12, 4), _moe(20, 8, 3, groups=4, keep=2, scale=1.3, limit=1.0)),
                   _layer(_attn(4, 1, 8, 16, 7, 5.0, 0.3), None),
                   _layer(_attn(4, 1, 8, 16, 7, 5.0, 0.3), _moe(12, 6, 2, groups=3, keep=1, scale=0.7, limit=0.5)),
                   _layer(_delta(2, 2, 24, 8, 2), None)]}
RANKS_A = {0: (5, 7), 3: (3, 2)}
# everything that can be 1, equal or absent: no streams key, one norm group, as many key heads as
# query heads, a chunk of exactly one page, no groups in the router, one expert per token, one
# convolution tap (no history), router scale 1
NX_B = {"architecture": "Notirax", "vocab": 64, "width": 32, "norm": {"eps": 1e-6},
        "layers": [_layer(_attn(2, 2, 16, 16, 16, 50.0), _moe(8, 4, 1)),
                   _layer(_delta(2, 2, 16, 16, 1), _moe(8, 4, 1)),
                   _layer(_attn(2, 2, 16, 16, 0, 0.0), _moe(16, 2, 2))]}
RANKS_B = {1: (4, 4)}
# still small, with the sizes the tensor-core kernels are written for: head sizes 64, chunks longer
# than a tile of keys, expert sizes of whole tiles, prompts of hundreds of tokens
NX_C = {"architecture": "Notirax", "vocab": 320, "width": 192, "streams": 4, "norm": {"eps": 1e-6, "groups": 2},
        "layers": [_layer(_attn(4, 2, 64, 64, 200, 20.0), _moe(64, 8, 2, groups=4, keep=3, scale=1.5)),
                   _layer(_delta(4, 2, 64, 32, 3), _moe(64, 8, 2, groups=2, keep=1, scale=1.5)),
                   _layer(_attn(4, 2, 64, 64, 200, 20.0), _moe(64, 8, 2, groups=4, keep=3, scale=1.5)),
                   _layer(_delta(4, 4, 32, 64, 3), None)]}
RANKS_C = {1: (16, 8), 3: (8, 16)}
CONFIGS = {"A": (NX_A, RANKS_A), "B": (NX_B, RANKS_B), "C": (NX_C, RANKS_C)}


def tensor_shapes(cfg, ranks):
    H, S = cfg["width"], cfg.get("streams")
    out = [("embed", (cfg["vocab"], H))]
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        nh, nkv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.append((p + "norm1", (H,)))
        if layer["type"] == "attention":
            for n, rows in (("q", nh * d), ("k", nkv * d), ("v", nkv * dv)):
                out += [(p + "mix." + n, (rows, H)), (p + "mix." + n + ".b", (rows,))]
            out += [(p + "mix.talk", (nh, nh)), (p + "mix.o", (H, nh * dv)), (p + "mix.o.b", (H,))]
        else:
            ra, rg = ranks[i]
            for n, rows in (("q", nkv * d), ("k", nkv * d), ("v", nh * dv)):
                out += [(p + "mix." + n, (rows, H)), (p + "mix." + n + ".conv", (rows, m["conv"]))]
            out += [(p + "mix.b", (nh, H)), (p + "mix.A_log", (nh,)), (p + "mix.norm", (dv,)),
                    (p + "mix.a1", (ra, H)), (p + "mix.a2", (nh * d, ra)), (p + "mix.dt_bias", (nh * d,)),
                    (p + "mix.g1", (rg, H)), (p + "mix.g2", (nh * dv, rg)), (p + "mix.o", (H, nh * dv))]
        mlp = layer["mlp"]
        if mlp is not None:
            out.append((p + "norm2", (H,)))
            for e in range(mlp["router"]["experts"]):
                out += [(f"{p}mlp.e{e}.gate", (mlp["expert"]["ff"], H)), (f"{p}mlp.e{e}.up", (mlp["expert"]["ff"], H)),
                        (f"{p}mlp.e{e}.down", (H, mlp["expert"]["ff"]))]
            out.append((p + "mlp.router", (mlp["router"]["experts"], H)))
        if S:
            for q in ("hc1",) + (("hc2",) if mlp is not None else ()):
                out += [(f"{p}{q}.in", (S,)), (f"{p}{q}.out", (S,)), (f"{p}{q}.mix", (S, S))]
    out.append(("final.norm", (H,)))
    return out


def random_weights(cfg, ranks, seed, qk_gain=1.0):
    """float32 arrays, exact in bfloat16.  ``qk_gain`` scales the attention's query and key
    projections so that the softmax is peaked and a wrong or missing key changes the logits."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, ranks):
        n = lambda std: rng.standard_normal(shape).astype(np.float32) * np.float32(std)
        leaf = name.split(".")[-1]
        if name == "embed":
            a = n(0.5)
        elif leaf in ("norm1", "norm2") or name in ("final.norm",) or name.endswith("mix.norm"):
            a = 1.0 + n(0.1)
        elif leaf == "in":
            a = 1.0 / shape[0] + n(0.1)
        elif leaf == "out":
            a = 1.0 + n(0.1)
        elif leaf == "mix":
            a = np.eye(shape[0], dtype=np.float32) + n(0.1)
        elif leaf == "talk":
            a = np.eye(shape[0], dtype=np.float32) + n(0.25)
        elif leaf == "conv":
            a = n(0.6)
        elif leaf in ("A_log", "dt_bias"):
            a = n(0.7)
        elif name.endswith(".b") and len(shape) == 1:
            a = n(0.2)
        elif leaf == "router":
            a = n(3.0 / np.sqrt(shape[1]))
        else:
            a = n(1.2 / np.sqrt(shape[1]))
            if ".mix.q" in name or ".mix.k" in name:
                layer = cfg["layers"][int(name[1:name.index(".")])]
                if layer["type"] == "attention":
                    a = a * np.float32(qk_gain)
        w[name] = bf16_round(a.astype(np.float32))
    return w


def make_model(tmp_path, which, seed=0, qk_gain=1.0):
    cfg, ranks = CONFIGS[which]
    w = random_weights(cfg, ranks, seed, qk_gain)
    d = write_model_dir(str(tmp_path / f"notirax_{which}_{seed}_{qk_gain}"), cfg, w, "bfloat16")
    return d, cfg, {k: v.astype(np.float64) for k, v in w.items()}


def prompt(cfg, n, seed):
    return np.random.default_rng(7000 + seed).integers(0, cfg["vocab"], size=n).tolist()
