"""Typed configuration of the Luzinex decoder, read from its own ``config.json`` keys.

    {"architecture": "Luzinex", "vocab": V, "width": H, "norm": {"eps": e},
     "layers": [{"type": "latent_attention" | "attention" | "retention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...]}

Mixer keys.  ``latent_attention``: ``heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
rot.base`` and optionally ``kv_from`` (the layer whose cached latent this one reads; that layer must
be an earlier latent layer with a cache of its own and equal ``kv_rank``, ``rot_dim`` and ``rot.base``).
``attention``: ``heads, kv_heads, dim, vdim, scale, rot.base, rot.dims`` and optionally
``mask.size`` with ``mask.keep_first`` (no mask: plain causal).  ``retention``: ``heads, dim, vdim,
decay`` (one number per head), ``rot.base, rot.dims``.  ``vdim`` absent: ``dim``; ``scale`` absent:
the usual inverse root of the query/key width; ``rot.dims`` absent: all rotated channels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .model_config import ConfigError, ModelConfig, _require, architecture_name
from .notirax_config import _obj, _opt, _positive, _req

MIXER_TYPES = ("latent_attention", "attention", "retention")


def _rot(m: Dict[str, Any], where: str, default_dims: int) -> Tuple[float, int]:
    rot = _obj(m, "rot", where)
    base = _req(rot, "base", float, where + "rot.")
    dims = _opt(rot, "dims", int, default_dims, where + "rot.")
    if not (base > 0 and math.isfinite(base)):
        raise ConfigError(f"config.json: field '{where}rot.base' must be positive, got {base}")
    if dims < 0 or dims % 2 or dims > default_dims:
        raise ConfigError(f"config.json: field '{where}rot.dims' must be even and between 0 and {default_dims}, got {dims}")
    return base, dims


def _parse_mixer(kind: str, m: Dict[str, Any], where: str) -> Dict[str, Any]:
    out = {"heads": _positive(_req(m, "heads", int, where), where + "heads"),
           "dim": _positive(_req(m, "dim", int, where), where + "dim")}
    out["vdim"] = _positive(_opt(m, "vdim", int, out["dim"], where), where + "vdim")
    if kind == "latent_attention":
        out["rot_dim"] = _req(m, "rot_dim", int, where)
        out["q_rank"] = _positive(_req(m, "q_rank", int, where), where + "q_rank")
        out["kv_rank"] = _positive(_req(m, "kv_rank", int, where), where + "kv_rank")
        out["scale"] = _opt(m, "scale", float, float(out["dim"] + out["rot_dim"]) ** -0.5, where)
        out["rot_base"], dims = _rot(m, where, out["rot_dim"])
        if out["rot_dim"] < 0 or out["rot_dim"] % 2 or dims != out["rot_dim"]:
            raise ConfigError(f"config.json: {where}rot_dim must be even and equal to {where}rot.dims")
        out["kv_from"] = _opt(m, "kv_from", int, -1, where)
    elif kind == "attention":
        out["kv_heads"] = _positive(_opt(m, "kv_heads", int, out["heads"], where), where + "kv_heads")
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of {where}kv_heads "
                              f"({out['kv_heads']})")
        if out["vdim"] != out["dim"]:
            raise ConfigError(f"config.json: {where}vdim ({out['vdim']}) must equal {where}dim ({out['dim']}): the "
                              f"values of this mixer are its keys")
        out["scale"] = _opt(m, "scale", float, float(out["dim"]) ** -0.5, where)
        out["rot_base"], out["rot_dims"] = _rot(m, where, out["dim"])
        mask = _obj(m, "mask", where, required=False)
        out["window"] = _opt(mask, "size", int, 0, where + "mask.")
        out["keep_first"] = _opt(mask, "keep_first", int, 0, where + "mask.")
        if out["window"] < 0 or out["keep_first"] < 0:
            raise ConfigError(f"config.json: {where}mask.size and mask.keep_first must not be negative")
    else:
        out["rot_base"], out["rot_dims"] = _rot(m, where, out["dim"])
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != out["heads"] or not all(
                isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            raise ConfigError(f"config.json: field '{where}decay' must list one number per head ({out['heads']})")
        out["decay"] = tuple(float(d) for d in decay)
    if "scale" in out and not math.isfinite(out["scale"]):
        raise ConfigError(f"config.json: field '{where}scale' must be finite")
    return out


def _parse_mlp(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    kind = _req(m, "kind", str, where)
    if kind != "dense":
        raise ConfigError(f"config.json: {where}kind '{kind}' is not supported (supported: dense)")
    return {"kind": kind, "ff": _positive(_req(m, "ff", int, where), where + "ff")}


@dataclass(frozen=True)
class LuzinexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    # per layer: {"type", "mixer": {...}, "mlp": {...} | None}, parsed and checked
    layers: Tuple[Dict[str, Any], ...] = field(default=(), compare=False)

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "LuzinexConfig":
        if not isinstance(j, dict):
            raise ConfigError("config.json: top level must be an object")
        arch = architecture_name(j)
        vocab = _positive(_require(j, "vocab", int), "vocab")
        width = _positive(_require(j, "width", int), "width")
        eps = _req(_obj(j, "norm", ""), "eps", float, "norm.")
        if not (eps >= 0.0 and math.isfinite(eps)):
            raise ConfigError(f"config.json: field 'norm.eps' must be non-negative, got {eps}")
        raw_layers = j.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: missing required field 'layers' (a list of layers)")
        layers = []
        for i, layer in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: field 'layers[{i}]' has wrong type: expected object")
            kind = _req(layer, "type", str, where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type '{kind}' is not supported (supported: "
                                  f"{', '.join(MIXER_TYPES)})")
            mixer = _parse_mixer(kind, _obj(layer, "mixer", where), where + "mixer.")
            if kind == "latent_attention" and mixer["kv_from"] >= 0:
                src = mixer["kv_from"]
                ok = src < i and layers[src]["type"] == "latent_attention" and layers[src]["mixer"]["kv_from"] < 0
                if not ok or any(layers[src]["mixer"][k] != mixer[k] for k in ("kv_rank", "rot_dim", "rot_base")):
                    raise ConfigError(f"config.json: {where}mixer.kv_from ({src}) must name an earlier latent_attention "
                                      f"layer that has keys of its own and the same kv_rank, rot_dim and rot.base")
            mlp = layer.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: field '{where}mlp' has wrong type: expected object or null")
            layers.append({"type": kind, "mixer": mixer,
                           "mlp": None if mlp is None else _parse_mlp(mlp, where + "mlp.")})
        return cls(architecture=arch, raw=dict(j), vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers))

    def to_json(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "layers": []}
        for layer in self.layers:
            m = layer["mixer"]
            mixer: Dict[str, Any] = {"heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"]}
            if layer["type"] == "latent_attention":
                mixer.update(rot_dim=m["rot_dim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=m["scale"],
                             rot={"base": m["rot_base"], "dims": m["rot_dim"]})
                if m["kv_from"] >= 0:
                    mixer["kv_from"] = m["kv_from"]
            elif layer["type"] == "attention":
                mixer.update(kv_heads=m["kv_heads"], scale=m["scale"], rot={"base": m["rot_base"], "dims": m["rot_dims"]})
                if m["window"]:
                    mixer["mask"] = {"size": m["window"], "keep_first": m["keep_first"]}
            else:
                mixer.update(decay=list(m["decay"]), rot={"base": m["rot_base"], "dims": m["rot_dims"]})
            mlp = layer["mlp"]
            out["layers"].append({"type": layer["type"], "mixer": mixer,
                                  "mlp": None if mlp is None else {"kind": mlp["kind"], "ff": mlp["ff"]}})
        return out
