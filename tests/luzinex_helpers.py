"""Small Luzinex configurations that differ in every size and option, random weights for them (made
here, not by the engine's random-weights mode) and model folders written by the tests' own writer."""
from __future__ import annotations

import numpy as np

from helpers import bf16_round, write_model_dir


def _latent(heads, dim, rot, vdim, q_rank, kv_rank, base, scale=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot}, "scale": (dim + rot) ** -0.5 if scale is None else scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _attn(heads, kv, dim, rot_dims, base, window=0, keep=0, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "rot": {"base": base, "dims": rot_dims},
         "scale": dim ** -0.5 if scale is None else scale}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    return {"type": "attention", "mixer": m}


def _ret(heads, dim, vdim, rot_dims, base, decay):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                                           "rot": {"base": base, "dims": rot_dims}}}


def _layer(mixer, ff):
    return dict(mixer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


# odd sizes everywhere: a latent lane 28 wide, key and value sizes that differ, rotations over a part of
# the head, a window shorter than a page that keeps three tokens, a layer without a feed-forward, a
# later latent layer with other heads that reads the first one's cache
LZ_A = {"architecture": "Luzinex", "vocab": 101, "width": 48, "norm": {"eps": 1e-5},
        "layers": [_layer(_latent(3, 8, 4, 12, 20, 24, 5000.0, 0.3), 20),
                   _layer(_attn(4, 2, 24, 8, 300.0, window=11, keep=3, scale=0.25), 36),
                   _layer(_ret(3, 12, 20, 8, 70000.0, (0.9, 0.99, 0.75)), None),
                   _layer(_latent(2, 16, 4, 8, 12, 24, 5000.0, 0.2, kv_from=0), 20),
                   _layer(_attn(2, 1, 16, 16, 10000.0, window=37, keep=17), 28)]}
# everything that can be 1, equal or absent: one head, no mask at all, a window of exactly one page that
# keeps nothing, a decay of exactly 1, rotations over the whole head, as many key heads as query heads
LZ_B = {"architecture": "Luzinex", "vocab": 64, "width": 32, "norm": {"eps": 1e-6},
        "layers": [_layer(_attn(1, 1, 16, 16, 10000.0), 16),
                   _layer(_ret(1, 16, 16, 16, 10000.0, (1.0,)), 16),
                   _layer(_latent(1, 16, 16, 16, 16, 16, 10000.0), 16),
                   _layer(_attn(2, 2, 16, 2, 50.0, window=16, keep=0), None),
                   _layer(_ret(2, 8, 8, 8, 100.0, (0.5, 0.996)), 8)]}
# still small, with the sizes the tensor-core kernels take: latent lanes 64 and 96 wide, head sizes 64 and
# 128, windows longer than a tile of keys and shorter than a split, prompts of hundreds of tokens
LZ_C = {"architecture": "Luzinex", "vocab": 320, "width": 192, "norm": {"eps": 1e-6},
        "layers": [_layer(_attn(4, 2, 64, 32, 20000.0, window=80, keep=5), 256),
                   _layer(_latent(4, 32, 16, 32, 64, 48, 100000.0), 256),
                   _layer(_ret(2, 64, 64, 64, 500000.0, (0.97, 0.999)), 256),
                   _layer(_attn(2, 1, 128, 64, 30000.0, window=200, keep=70), 256),
                   _layer(_latent(2, 64, 16, 48, 32, 48, 100000.0, kv_from=1), 256),
                   _layer(_latent(6, 16, 32, 16, 48, 64, 777.0), None)]}
CONFIGS = {"A": LZ_A, "B": LZ_B, "C": LZ_C}


def tensor_shapes(cfg):
    H = cfg["width"]
    out = [("embed", (cfg["vocab"], H))]
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        nh, d, dv = m["heads"], m["dim"], m["vdim"]
        out.append((p + "norm1", (H,)))
        if layer["mlp"] is not None:
            out.append((p + "norm2", (H,)))
        if layer["type"] == "latent_attention":
            r, qr, kr = m["rot_dim"], m["q_rank"], m["kv_rank"]
            out += [(p + "mix.dq", (qr, H)), (p + "mix.dq.norm", (qr,)), (p + "mix.uq", (nh * (d + r), qr))]
            if "kv_from" not in m:
                out += [(p + "mix.dkv", (kr + r, H)), (p + "mix.dkv.norm", (kr,))]
            out += [(p + "mix.uk", (nh * d, kr)), (p + "mix.uv", (nh * dv, kr)), (p + "mix.g", (nh * dv, H)),
                    (p + "mix.o", (H, nh * dv))]
        elif layer["type"] == "attention":
            out += [(p + "mix.q", (nh * d, H)), (p + "mix.k", (m["kv_heads"] * d, H)), (p + "mix.sink", (nh,)),
                    (p + "mix.g", (nh * d, H)), (p + "mix.o", (H, nh * d))]
        else:
            out += [(p + "mix.q", (nh * d, H)), (p + "mix.k", (nh * d, H)), (p + "mix.v", (nh * dv, H)),
                    (p + "mix.g", (nh * dv, H)), (p + "mix.o", (H, nh * dv))]
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            out += [(p + "mlp.gate", (ff, H)), (p + "mlp.up", (ff, H)), (p + "mlp.down", (H, ff))]
    out += [("final.norm", (H,)), ("head", (cfg["vocab"], H))]
    return out


def random_weights(cfg, seed, qk_gain=1.0):
    """float32 arrays, exact in bfloat16.  ``qk_gain`` scales what makes queries and keys (the attention's
    q and k, the latent's uq and uk) so that the softmax is peaked and a wrong or missing key shows."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg):
        n = lambda std: rng.standard_normal(shape).astype(np.float32) * np.float32(std)
        leaf = name.split(".")[-1]
        if name == "embed":
            a = n(0.5)
        elif leaf in ("norm1", "norm2", "norm"):
            a = 1.0 + n(0.1)
        elif leaf == "sink":
            a = n(1.0)
        else:
            a = n(1.2 / np.sqrt(shape[1]))
            layer = cfg["layers"][int(name[1:name.index(".")])] if name[0] == "l" and name[1].isdigit() else None
            if layer is not None and layer["type"] != "retention" and leaf in ("q", "k", "uq", "uk"):
                a = a * np.float32(qk_gain)
        w[name] = bf16_round(a.astype(np.float32))
    return w


def make_model(tmp_path, which, seed=0, qk_gain=1.0):
    cfg = CONFIGS[which]
    w = random_weights(cfg, seed, qk_gain)
    d = write_model_dir(str(tmp_path / f"luzinex_{which}_{seed}_{qk_gain}"), cfg, w, "bfloat16")
    return d, cfg, {k: v.astype(np.float64) for k, v in w.items()}


def prompt(cfg, n, seed):
    return np.random.default_rng(9000 + seed).integers(0, cfg["vocab"], size=n).tolist()
