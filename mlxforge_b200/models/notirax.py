"""``Notirax``: a decoder whose layers are either attention with talking heads over chunks or a
gated delta rule with channel-wise decay, each followed by a mixture of experts (or by nothing),
joined to several residual streams by hyper-connections, with grouped RMS norms and sinusoidal
positions added to the embedding.  Described as data: every part is a registry kind that gets its
sizes and constants as parameters.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.mix.*`` (the mixer) and ``l<i>.mlp.router``, ``l<i>.mlp.e<k>.gate|up|down``.  The output head
is the embedding table.
"""
from __future__ import annotations

from typing import Iterator, Tuple

from ..config.notirax_config import NotiraxConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem


def build_notirax_spec(cfg: NotiraxConfig) -> ModelSpec:
    S = cfg.streams or 1
    H = cfg.width

    def norm(name: str) -> PartSpec:
        i = name.rindex(".") + 1 if "." in name else 0
        return PartSpec("group_rmsnorm", {"size": H, "eps": cfg.norm_eps, "groups": cfg.norm_groups, "streams": S,
                                          "tensor": name[i:]}, prefix=name[:i])

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixer = PartSpec("talking_attention", {
                "hidden_size": H, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "softmax_scale": m["scale"], "softcap": m["softcap"], "talking": True,
                "chunk": m["chunk"], "bias": True}, prefix=p + "mix.")
        else:
            if m["decay_rank"] <= 0 or m["gate_rank"] <= 0:
                raise ValueError(f"layer {i}: the low-rank sizes of the channel-delta mixer are unknown (they come from "
                                 f"the shapes of {p}mix.a1 and {p}mix.g1, or from mixer.decay_rank / mixer.gate_rank)")
            mixer = PartSpec("channel_delta", {
                "hidden_size": H, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "conv": m["conv"], "eps": cfg.norm_eps, "decay_rank": m["decay_rank"],
                "gate_rank": m["gate_rank"]}, prefix=p + "mix.")
        extra = []
        if cfg.streams:
            extra.append(("mixer_connection", "connection", PartSpec("hyper", {"streams": S}, prefix=p + "hc1.")))
        ff = ff_norm = None
        mlp = layer["mlp"]
        if mlp is not None:
            ff = PartSpec("routed_experts", {
                "hidden_size": H, "intermediate_size": mlp["ff"], "n_experts": mlp["experts"], "top": mlp["top"],
                "n_groups": mlp["groups"], "keep_groups": mlp["keep"], "route_scale": mlp["scale"],
                "limit": mlp["limit"], "alpha": 1.702}, prefix=p + "mlp.")
            ff_norm = norm(p + "norm2")
            if cfg.streams:
                extra.append(("feed_forward_connection", "connection",
                              PartSpec("hyper", {"streams": S}, prefix=p + "hc2.")))
        layers.append(LayerSpec(block="stream_prenorm", mixer=mixer, mixer_norm=norm(p + "norm1"), feed_forward=ff,
                                feed_forward_norm=ff_norm, extra=tuple(extra)))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "embed",
                                               "positions": "sinusoid", "theta": 10000.0}),
        layers=tuple(layers), schedule=tuple(ScheduleItem(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "head", "tied_to": "embed",
                                      "require_own": False}),
        streams=S,
    )


def notirax_random_tensors(cfg: NotiraxConfig) -> Iterator[Tuple[str, Tuple[int, ...], object]]:
    """Names, shapes and kinds of a checkpoint of this configuration, in file order.  A kind is
    ``matrix``, ``norm`` or ``(mean, std)`` of a normal draw; ``("eye", std)`` is the identity plus noise."""
    H, S = cfg.width, cfg.streams
    yield "embed", (cfg.vocab, H), "matrix"
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        nh, nkv, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        yield p + "norm1", (H,), "norm"
        if layer["mlp"] is not None:
            yield p + "norm2", (H,), "norm"
        if layer["type"] == "attention":
            for n, rows in (("q", nh * d), ("k", nkv * d), ("v", nkv * dv)):
                yield p + "mix." + n, (rows, H), "matrix"
                yield p + "mix." + n + ".b", (rows,), (0.0, 0.02)
            yield p + "mix.talk", (nh, nh), ("eye", 0.1)
            yield p + "mix.o", (H, nh * dv), "matrix"
            yield p + "mix.o.b", (H,), (0.0, 0.02)
        else:
            for n, rows in (("q", nkv * d), ("k", nkv * d), ("v", nh * dv)):
                yield p + "mix." + n, (rows, H), "matrix"
                yield p + "mix." + n + ".conv", (rows, m["conv"]), (0.0, 0.5)
            yield p + "mix.b", (nh, H), "matrix"
            yield p + "mix.A_log", (nh,), (0.0, 0.5)
            yield p + "mix.norm", (dv,), "norm"
            yield p + "mix.a1", (m["decay_rank"], H), "matrix"
            yield p + "mix.a2", (nh * d, m["decay_rank"]), "matrix"
            yield p + "mix.dt_bias", (nh * d,), (0.0, 0.5)
            yield p + "mix.g1", (m["gate_rank"], H), "matrix"
            yield p + "mix.g2", (nh * dv, m["gate_rank"]), "matrix"
            yield p + "mix.o", (H, nh * dv), "matrix"
        mlp = layer["mlp"]
        if mlp is not None:
            for e in range(mlp["experts"]):
                yield f"{p}mlp.e{e}.gate", (mlp["ff"], H), "matrix"
                yield f"{p}mlp.e{e}.up", (mlp["ff"], H), "matrix"
                yield f"{p}mlp.e{e}.down", (H, mlp["ff"]), "matrix"
            yield p + "mlp.router", (mlp["experts"], H), "matrix"
        if S:
            for q in ("hc1",) + (("hc2",) if mlp is not None else ()):
                yield f"{p}{q}.in", (S,), (1.0 / S, 0.05)
                yield f"{p}{q}.out", (S,), (1.0, 0.05)
                yield f"{p}{q}.mix", (S, S), ("eye", 0.05)
    yield "final.norm", (H,), "norm"


register_architecture("Notirax", NotiraxConfig, build_notirax_spec, notirax_random_tensors, replace=True)
