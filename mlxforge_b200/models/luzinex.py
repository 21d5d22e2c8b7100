"""``Luzinex``: a decoder whose layers run their mixer and their feed-forward side by side on one
residual, each behind an RMS norm of its own.  The mixers, in an order that config.json gives, are
attention over a compressed latent (a later layer may read an earlier one's cache), grouped-query
attention whose values are its keys, with a sliding window that keeps the first tokens, a sink in
the softmax and a gate on the output, and retention with a fixed decay per head; the feed-forward
is dense and gated with the tanh form of GELU.  Described as data: every part is a registry kind
that gets its sizes and constants as parameters.

Tensor names: ``embed``, ``final.norm``, ``head``, and per layer ``l<i>.norm1|norm2``,
``l<i>.mix.*`` (the mixer) and ``l<i>.mlp.gate|up|down``.
"""
from __future__ import annotations

from typing import Iterator, Tuple

from ..config.luzinex_config import LuzinexConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem


def build_luzinex_spec(cfg: LuzinexConfig) -> ModelSpec:
    H = cfg.width

    def norm(name: str) -> PartSpec:
        i = name.rindex(".") + 1
        return PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": name[i:]}, prefix=name[:i])

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        cache_of = None
        if layer["type"] == "latent_attention":
            shares = m["kv_from"] >= 0
            cache_of = m["kv_from"] if shares else None
            mixer = PartSpec("latent_attention", {
                "hidden_size": H, "n_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "v_head_dim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "softmax_scale": m["scale"],
                "rope_base": m["rot_base"], "eps": cfg.norm_eps, "gate": True, "shares_cache": shares},
                prefix=p + "mix.")
        elif layer["type"] == "attention":
            mixer = PartSpec("sink_attention", {
                "hidden_size": H, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "softmax_scale": m["scale"], "window": m["window"], "keep_first": m["keep_first"], "values": "keys",
                "sink": True, "gate": True,
                "position": PartSpec("rotary", {"head_dim": m["dim"], "rotary_dim": m["rot_dims"],
                                                "base": m["rot_base"], "pairing": "pairs"})}, prefix=p + "mix.")
        else:
            mixer = PartSpec("retention", {
                "hidden_size": H, "n_heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
                "rotary_dim": m["rot_dims"], "rope_base": m["rot_base"], "decay": tuple(m["decay"]),
                "eps": cfg.norm_eps}, prefix=p + "mix.")
        ff = ff_norm = None
        if layer["mlp"] is not None:
            ff = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": layer["mlp"]["ff"],
                                     "activation": "gelu_tanh",
                                     "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix=p + "mlp.")
            ff_norm = norm(p + "norm2")
        layers.append(LayerSpec(block="parallel", mixer=mixer, mixer_norm=norm(p + "norm1"), feed_forward=ff,
                                feed_forward_norm=ff_norm))
        # every layer runs once, in order, so a layer's index is also its place in the schedule
        schedule.append(ScheduleItem(i, cache_of=cache_of))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "embed"}),
        layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tensor": "head",
                                      "require_own": True}),
    )


def luzinex_random_tensors(cfg: LuzinexConfig) -> Iterator[Tuple[str, Tuple[int, ...], object]]:
    """Names, shapes and kinds of a checkpoint of this configuration, in file order."""
    H = cfg.width
    yield "embed", (cfg.vocab, H), "matrix"
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        nh, d, dv = m["heads"], m["dim"], m["vdim"]
        yield p + "norm1", (H,), "norm"
        if layer["mlp"] is not None:
            yield p + "norm2", (H,), "norm"
        if layer["type"] == "latent_attention":
            yield p + "mix.dq", (m["q_rank"], H), "matrix"
            yield p + "mix.dq.norm", (m["q_rank"],), "norm"
            yield p + "mix.uq", (nh * (d + m["rot_dim"]), m["q_rank"]), "matrix"
            if m["kv_from"] < 0:
                yield p + "mix.dkv", (m["kv_rank"] + m["rot_dim"], H), "matrix"
                yield p + "mix.dkv.norm", (m["kv_rank"],), "norm"
            yield p + "mix.uk", (nh * d, m["kv_rank"]), "matrix"
            yield p + "mix.uv", (nh * dv, m["kv_rank"]), "matrix"
            yield p + "mix.g", (nh * dv, H), "matrix"
            yield p + "mix.o", (H, nh * dv), "matrix"
        elif layer["type"] == "attention":
            yield p + "mix.q", (nh * d, H), "matrix"
            yield p + "mix.k", (m["kv_heads"] * d, H), "matrix"
            yield p + "mix.sink", (nh,), (0.0, 1.0)
            yield p + "mix.g", (nh * d, H), "matrix"
            yield p + "mix.o", (H, nh * d), "matrix"
        else:
            yield p + "mix.q", (nh * d, H), "matrix"
            yield p + "mix.k", (nh * d, H), "matrix"
            yield p + "mix.v", (nh * dv, H), "matrix"
            yield p + "mix.g", (nh * dv, H), "matrix"
            yield p + "mix.o", (H, nh * dv), "matrix"
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            yield p + "mlp.gate", (ff, H), "matrix"
            yield p + "mlp.up", (ff, H), "matrix"
            yield p + "mlp.down", (H, ff), "matrix"
    yield "final.norm", (H,), "norm"
    yield "head", (cfg.vocab, H), "matrix"


register_architecture("Luzinex", LuzinexConfig, build_luzinex_spec, luzinex_random_tensors, replace=True)
