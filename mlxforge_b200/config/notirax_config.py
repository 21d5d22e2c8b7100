"""Typed configuration of the Notirax decoder, read from its own ``config.json`` keys.

    {"architecture": "Notirax", "vocab": V, "width": H, "streams": S,
     "norm": {"eps": e, "groups": G},
     "layers": [{"type": "attention" | "channel_delta", "mixer": {...}, "mlp": {...} | null}, ...]}

``streams`` absent: one residual stream.  ``norm.groups`` absent: one group.  An attention mixer
has ``heads, kv_heads, dim, vdim, scale, softcap, mask.size``; a channel-delta mixer
``heads, kv_heads, dim, vdim, conv``; a feed-forward ``kind: "moe"`` with ``expert.ff, expert.limit``
and ``router.experts, router.top, router.scale, router.groups.count, router.groups.keep``.  The two
low-rank sizes of a channel-delta mixer are not in config.json: they are the first extent of the
tensors ``l<i>.mix.a1`` and ``l<i>.mix.g1`` (``with_tensor_shapes``); a configuration that is to be
written with random weights names them as ``mixer.decay_rank`` and ``mixer.gate_rank``.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .model_config import ConfigError, ModelConfig, _optional, _require, architecture_name

MIXER_TYPES = ("attention", "channel_delta")


def _obj(j: Dict[str, Any], key: str, where: str, required: bool = True) -> Dict[str, Any]:
    v = j.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: missing required field '{where}{key}'")
        return {}
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: field '{where}{key}' has wrong type: expected object, got {type(v).__name__}")
    return v


def _req(j, key, kind, where):
    try:
        return _require(j, key, kind)
    except ConfigError as e:
        raise ConfigError(str(e).replace(f"'{key}'", f"'{where}{key}'")) from None


def _opt(j, key, kind, default, where):
    try:
        return _optional(j, key, kind, default)
    except ConfigError as e:
        raise ConfigError(str(e).replace(f"'{key}'", f"'{where}{key}'")) from None


def _positive(v, name):
    if v <= 0:
        raise ConfigError(f"config.json: field '{name}' must be positive, got {v}")
    return v


def _parse_mixer(kind: str, m: Dict[str, Any], where: str) -> Dict[str, Any]:
    out = {
        "heads": _positive(_req(m, "heads", int, where), where + "heads"),
        "kv_heads": _positive(_req(m, "kv_heads", int, where), where + "kv_heads"),
        "dim": _positive(_req(m, "dim", int, where), where + "dim"),
    }
    out["vdim"] = _positive(_opt(m, "vdim", int, out["dim"], where), where + "vdim")
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of {where}kv_heads "
                          f"({out['kv_heads']})")
    if kind == "attention":
        out["scale"] = _opt(m, "scale", float, float(out["dim"]) ** -0.5, where)
        out["softcap"] = _opt(m, "softcap", float, 0.0, where)
        mask = _obj(m, "mask", where, required=False)
        out["chunk"] = _opt(mask, "size", int, 0, where + "mask.")
        if not math.isfinite(out["scale"]) or out["softcap"] < 0 or out["chunk"] < 0:
            raise ConfigError(f"config.json: {where}scale, softcap and mask.size must be finite and not negative")
    else:
        out["conv"] = _positive(_req(m, "conv", int, where), where + "conv")
        out["decay_rank"] = _opt(m, "decay_rank", int, 0, where)
        out["gate_rank"] = _opt(m, "gate_rank", int, 0, where)
    return out


def _parse_mlp(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    kind = _req(m, "kind", str, where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}kind '{kind}' is not supported (supported: moe)")
    ex = _obj(m, "expert", where)
    ro = _obj(m, "router", where)
    gr = _obj(ro, "groups", where + "router.", required=False)
    out = {
        "kind": kind,
        "ff": _positive(_req(ex, "ff", int, where + "expert."), where + "expert.ff"),
        "limit": _req(ex, "limit", float, where + "expert."),
        "experts": _positive(_req(ro, "experts", int, where + "router."), where + "router.experts"),
        "top": _positive(_req(ro, "top", int, where + "router."), where + "router.top"),
        "scale": _opt(ro, "scale", float, 1.0, where + "router."),
        "groups": _opt(gr, "count", int, 0, where + "router.groups."),
        "keep": _opt(gr, "keep", int, 0, where + "router.groups."),
    }
    if out["top"] > out["experts"]:
        raise ConfigError(f"config.json: {where}router.top ({out['top']}) exceeds router.experts ({out['experts']})")
    if out["groups"]:
        if out["experts"] % out["groups"] or not (1 <= out["keep"] <= out["groups"]):
            raise ConfigError(f"config.json: {where}router.groups does not fit {out['experts']} experts")
        if out["keep"] * (out["experts"] // out["groups"]) < out["top"]:
            raise ConfigError(f"config.json: {where}router.groups keeps fewer experts than router.top")
    return out


@dataclass(frozen=True)
class NotiraxConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    streams: int = 0                 # 0: config.json names none (one ordinary residual stream)
    norm_eps: float = 0.0
    norm_groups: int = 1
    # per layer: {"type", "mixer": {...}, "mlp": {...} | None}, parsed and checked
    layers: Tuple[Dict[str, Any], ...] = field(default=(), compare=False)

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "NotiraxConfig":
        if not isinstance(j, dict):
            raise ConfigError("config.json: top level must be an object")
        arch = architecture_name(j)
        vocab = _positive(_require(j, "vocab", int), "vocab")
        width = _positive(_require(j, "width", int), "width")
        streams = _optional(j, "streams", int, 0)
        if streams < 0 or streams > 8:
            raise ConfigError(f"config.json: field 'streams' must be between 1 and 8, got {streams}")
        norm = _obj(j, "norm", "")
        eps = _req(norm, "eps", float, "norm.")
        groups = _opt(norm, "groups", int, 1, "norm.")
        if not (eps >= 0.0 and math.isfinite(eps)):
            raise ConfigError(f"config.json: field 'norm.eps' must be non-negative, got {eps}")
        if groups < 1 or width % groups:
            raise ConfigError(f"config.json: field 'norm.groups' ({groups}) must divide 'width' ({width})")
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
            mlp = layer.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: field '{where}mlp' has wrong type: expected object or null")
            layers.append({"type": kind, "mixer": mixer,
                           "mlp": None if mlp is None else _parse_mlp(mlp, where + "mlp.")})
        return cls(architecture=arch, raw=dict(j), vocab=vocab, width=width, streams=streams, norm_eps=eps,
                   norm_groups=groups, layers=tuple(layers))

    def with_tensor_shapes(self, shapes: Dict[str, tuple]) -> "NotiraxConfig":
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            if layer["type"] != "channel_delta":
                continue
            for key, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                if name in shapes and len(shapes[name]) == 2:
                    layer["mixer"][key] = int(shapes[name][0])
        return NotiraxConfig(architecture=self.architecture, raw=self.raw, vocab=self.vocab, width=self.width,
                             streams=self.streams, norm_eps=self.norm_eps, norm_groups=self.norm_groups,
                             layers=tuple(layers))

    def to_json(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": []}
        if self.streams:
            out["streams"] = self.streams
        for layer in self.layers:
            m = layer["mixer"]
            mixer = {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"]}
            if layer["type"] == "attention":
                mixer.update(scale=m["scale"], softcap=m["softcap"])
                if m["chunk"]:
                    mixer["mask"] = {"size": m["chunk"]}
            else:
                mixer.update(conv=m["conv"], decay_rank=m["decay_rank"], gate_rank=m["gate_rank"])
            mlp = layer["mlp"]
            if mlp is not None:
                router = {"experts": mlp["experts"], "top": mlp["top"], "scale": mlp["scale"]}
                if mlp["groups"]:
                    router["groups"] = {"count": mlp["groups"], "keep": mlp["keep"]}
                mlp = {"kind": mlp["kind"], "expert": {"ff": mlp["ff"], "limit": mlp["limit"]}, "router": router}
            out["layers"].append({"type": layer["type"], "mixer": mixer, "mlp": mlp})
        return out
