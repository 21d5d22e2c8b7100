"""CPU tests of the Notirax pieces that need no device: the plain implementation against closed
forms and against itself, the configuration reader, the tensor list of the random-weights mode,
and the cache manager's page discipline under a chunk-local mask."""
import json

import numpy as np
import pytest

import plain_llama as PL
import plain_notirax as P
from notirax_helpers import CONFIGS, NX_A, NX_B, RANKS_A, random_weights, tensor_shapes


# ----------------------------------------------------------------------------- the plain implementation

def test_sinusoid_closed_form():
    pe = P.sinusoid([0, 1, 5], 6)
    assert np.allclose(pe[0], [0, 1, 0, 1, 0, 1])
    f = [1.0, 10000.0 ** (-2 / 6), 10000.0 ** (-4 / 6)]
    assert np.allclose(pe[2], [np.sin(5 * f[0]), np.cos(5 * f[0]), np.sin(5 * f[1]), np.cos(5 * f[1]),
                               np.sin(5 * f[2]), np.cos(5 * f[2])])


def test_group_norm_with_one_group_is_rmsnorm_and_groups_are_independent():
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((5, 12)), rng.standard_normal(12)
    assert np.allclose(P.group_rms_norm(x, w, 1e-5, 1), PL.rms_norm(x, w, 1e-5))
    y = P.group_rms_norm(x, np.ones(12), 0.0, 3)
    assert np.allclose((y.reshape(5, 3, 4) ** 2).mean(-1), 1.0)
    x2 = x.copy()
    x2[:, 8:] *= 100.0                      # another group's size changes nothing here
    assert np.allclose(P.group_rms_norm(x2, w, 1e-5, 3)[:, :8], P.group_rms_norm(x, w, 1e-5, 3)[:, :8])


def test_hyper_streams_with_one_stream_are_the_residual_sum():
    rng = np.random.default_rng(1)
    x, y = rng.standard_normal((1, 4, 6)), rng.standard_normal((4, 6))
    assert np.allclose(P.hyper_read(x, np.ones(1)), x[0])
    assert np.allclose(P.hyper_write(x, y, np.ones((1, 1)), np.ones(1))[0], x[0] + y)
    # mix is [from, to]: stream 0 flows into stream 1 only
    s = rng.standard_normal((2, 4, 6))
    mix = np.array([[0.0, 1.0], [0.0, 0.0]])
    out = P.hyper_write(s, np.zeros((4, 6)), mix, np.zeros(2))
    assert np.allclose(out[1], s[0]) and np.allclose(out[0], 0)


def _attn_weights(rng, H, nh, nkv, d, dv, talk=None):
    w = {"q": rng.standard_normal((nh * d, H)), "k": rng.standard_normal((nkv * d, H)),
         "v": rng.standard_normal((nkv * dv, H)), "o": rng.standard_normal((H, nh * dv)),
         "q.b": np.zeros(nh * d), "k.b": np.zeros(nkv * d), "v.b": np.zeros(nkv * dv), "o.b": np.zeros(H)}
    if talk is not None:
        w["talk"] = talk
    return w


def test_talking_attention_reduces_to_plain_attention():
    """Identity mixing, no cap, no chunk: the plain causal GQA attention of the other oracle."""
    rng = np.random.default_rng(2)
    H, nh, nkv, d = 20, 4, 2, 6
    w = _attn_weights(rng, H, nh, nkv, d, d, talk=np.eye(nh))
    h = rng.standard_normal((9, H))
    p = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": d, "scale": d ** -0.5}
    got = P.talking_chunk_attention(h, p, w.get)
    q, k, v = PL.project_qkv(h, w["q"], w["k"], w["v"], nh, nkv, d)
    want = PL.attention(q, k, v, d ** -0.5, 0) @ w["o"].T
    assert np.allclose(got, want)


def test_chunk_mask_softcap_and_talk_by_hand():
    rng = np.random.default_rng(3)
    H, nh, d, dv, T, size = 10, 2, 4, 3, 7, 3
    talk = np.array([[0.5, 2.0], [-1.0, 1.0]])
    w = _attn_weights(rng, H, nh, 1, d, dv, talk=talk)
    for n in ("q.b", "k.b", "v.b", "o.b"):
        w[n] = rng.standard_normal(w[n].shape)
    h = rng.standard_normal((T, H))
    p = {"heads": nh, "kv_heads": 1, "dim": d, "vdim": dv, "scale": 0.7, "softcap": 2.0, "mask": {"size": size}}
    got = P.talking_chunk_attention(h, p, w.get)
    q = (h @ w["q"].T + w["q.b"]).reshape(T, nh, d)
    k = h @ w["k"].T + w["k.b"]
    v = h @ w["v"].T + w["v.b"]
    o = np.zeros((T, nh, dv))
    for i in range(T):
        js = [j for j in range(i + 1) if j // size == i // size]
        raw = np.array([[2.0 * np.tanh(q[i, a] @ k[j] * 0.7 / 2.0) for j in js] for a in range(nh)])
        mixed = talk @ raw
        for a in range(nh):
            e = np.exp(mixed[a] - mixed[a].max())
            o[i, a] = (e / e.sum()) @ v[js]
    assert np.allclose(got, o.reshape(T, -1) @ w["o"].T + w["o.b"])
    # the first token of a chunk sees itself only
    assert np.allclose(o[size], np.repeat(v[size][None], nh, axis=0))


def _delta_weights(rng, H, nh, nkv, d, dv, taps, ra=3, rg=2):
    return {"q": rng.standard_normal((nkv * d, H)), "k": rng.standard_normal((nkv * d, H)),
            "v": rng.standard_normal((nh * dv, H)), "q.conv": rng.standard_normal((nkv * d, taps)),
            "k.conv": rng.standard_normal((nkv * d, taps)), "v.conv": rng.standard_normal((nh * dv, taps)),
            "b": rng.standard_normal((nh, H)), "A_log": rng.standard_normal(nh) * 0.3,
            "dt_bias": rng.standard_normal(nh * d), "a1": rng.standard_normal((ra, H)),
            "a2": rng.standard_normal((nh * d, ra)), "g1": rng.standard_normal((rg, H)),
            "g2": rng.standard_normal((nh * dv, rg)), "norm": 1 + 0.1 * rng.standard_normal(dv),
            "o": rng.standard_normal((H, nh * dv))}


def test_short_conv_by_hand():
    x = np.arange(10.0).reshape(5, 2)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = P.short_conv(x, w)
    assert np.allclose(y[:, 1], x[:, 1])                               # the last tap is the current token's
    assert np.allclose(y[0, 0], 100 * x[0, 0]) and np.allclose(y[2, 0], x[0, 0] + 10 * x[1, 0] + 100 * x[2, 0])


def test_channel_delta_is_causal_and_its_first_token_is_closed_form():
    rng = np.random.default_rng(4)
    H, nh, nkv, d, dv, taps = 12, 4, 2, 5, 3, 3
    w = _delta_weights(rng, H, nh, nkv, d, dv, taps)
    p = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": dv, "conv": taps}
    h = rng.standard_normal((8, H))
    full = P.channel_delta(h, p, w.get, 1e-6)
    assert np.allclose(P.channel_delta(h[:5], p, w.get, 1e-6), full[:5])
    # token 0: S = k u^T with u = beta v, so o = (k . q) beta v per head
    x = h[:1]
    q = P.silu(x @ w["q"].T * w["q.conv"][:, -1]).reshape(nkv, d)
    k = P.silu(x @ w["k"].T * w["k.conv"][:, -1]).reshape(nkv, d)
    v = P.silu(x @ w["v"].T * w["v.conv"][:, -1]).reshape(nh, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) / np.sqrt(d)
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = P.sigmoid(x @ w["b"].T)[0]
    o = np.stack([(k[a // 2] @ q[a // 2]) * beta[a] * v[a] for a in range(nh)])
    o = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-6) * w["norm"]
    gate = P.sigmoid((x @ w["g1"].T) @ w["g2"].T).reshape(nh, dv)
    assert np.allclose(full[0], (o * gate).reshape(-1) @ w["o"].T)


def test_delta_rule_with_full_decay_forgets_and_with_none_keeps():
    """g -> 0 (huge dt_bias): every token only sees its own write; the decay multiplies rows of S."""
    rng = np.random.default_rng(5)
    H, nh, d, dv = 6, 1, 4, 3
    w = _delta_weights(rng, H, nh, 1, d, dv, 1)
    p = {"heads": nh, "kv_heads": 1, "dim": d, "vdim": dv, "conv": 1}
    h = rng.standard_normal((6, H))
    w["dt_bias"] = np.full(nh * d, 60.0)
    forget = P.channel_delta(h, p, w.get, 1e-6)
    alone = np.concatenate([P.channel_delta(h[t:t + 1], p, w.get, 1e-6) for t in range(6)])
    assert np.allclose(forget, alone)
    w["dt_bias"] = np.full(nh * d, -60.0)
    keep = P.channel_delta(h, p, w.get, 1e-6)
    assert not np.allclose(keep[1:], alone[1:])


def test_grouped_router_by_hand():
    # 6 experts in 3 groups of 2; logits chosen so that the best single expert sits in a group that loses
    z = np.array([[4.0, -9.0, 2.0, 2.5, 1.0, 3.0]])
    s = P.sigmoid(z)
    r = {"top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    chosen, weight = P.grouped_router(z, np.eye(6), r)
    # group scores: s0+s1 ~ 0.98, s2+s3 ~ 1.80, s4+s5 ~ 1.68 -> group 1 stays, expert 0 cannot be chosen
    assert chosen.tolist() == [[3, 2]]
    assert np.allclose(weight, 2.0 * s[:, [3, 2]])
    chosen, _ = P.grouped_router(z, np.eye(6), {"top": 2, "scale": 1.0})
    assert chosen.tolist() == [[0, 5]]
    chosen, _ = P.grouped_router(z, np.eye(6), {"top": 3, "scale": 1.0, "groups": {"count": 3, "keep": 2}})
    assert chosen.tolist() == [[5, 3, 2]]


def test_clamped_expert_by_hand():
    h = np.array([[1.0, -2.0]])
    wg, wu, wd = np.array([[3.0, 0.0], [0.0, 1.0]]), np.array([[0.0, 2.0], [1.0, 0.0]]), np.array([[1.0, 1.0]])
    g = np.minimum(np.array([3.0, -2.0]), 1.5)
    u = np.clip(np.array([-4.0, 1.0]), -1.5, 1.5)
    want = (g * P.sigmoid(1.702 * g) * (u + 1)).sum()
    assert np.allclose(P.clamped_expert(h, wg, wu, wd, 1.5), want)


@pytest.mark.parametrize("which", ["A", "B"])
def test_whole_model_is_causal(which):
    cfg, ranks = CONFIGS[which]
    w = {k: v.astype(np.float64) for k, v in random_weights(cfg, ranks, 1).items()}
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], size=40).tolist()
    layers = []
    full = P.forward(cfg, w, toks, layers)
    assert len(layers) == len(cfg["layers"]) and np.isfinite(full).all()
    assert np.allclose(P.forward(cfg, w, toks[:23]), full[:23])


# ----------------------------------------------------------------------------- configuration

def test_config_reader_keys_defaults_and_errors():
    from mlxforge_b200.config import ConfigError, NotiraxConfig, config_from_json
    c = config_from_json(json.loads(json.dumps(NX_A)))
    assert isinstance(c, NotiraxConfig) and (c.vocab, c.width, c.streams, c.norm_groups) == (101, 48, 2, 3)
    assert c.layers[1]["mixer"]["chunk"] == 7 and c.layers[1]["mlp"] is None
    assert c.layers[0]["mlp"]["groups"] == 4 and c.layers[0]["mlp"]["keep"] == 2
    b = config_from_json(json.loads(json.dumps(NX_B)))
    assert b.streams == 0 and b.norm_groups == 1 and b.layers[2]["mixer"]["chunk"] == 0
    assert b.layers[0]["mlp"]["groups"] == 0 and b.layers[0]["mlp"]["scale"] == 1.0
    # the low-rank sizes come from tensor shapes
    c2 = c.with_tensor_shapes({"l0.mix.a1": (5, 48), "l0.mix.g1": (7, 48), "l3.mix.a1": (3, 48), "l3.mix.g1": (2, 48)})
    assert (c2.layers[0]["mixer"]["decay_rank"], c2.layers[0]["mixer"]["gate_rank"]) == (5, 7)
    assert config_from_json(c2.to_json()).to_json() == c2.to_json()

    def broken(edit, text):
        j = json.loads(json.dumps(NX_A))
        edit(j)
        with pytest.raises(ConfigError, match=text):
            config_from_json(j)
    broken(lambda j: j.pop("width"), "missing required field 'width'")
    broken(lambda j: j["norm"].pop("eps"), "norm.eps")
    broken(lambda j: j["layers"][0].update(type="conv"), "not supported")
    broken(lambda j: j["layers"][1]["mixer"].update(kv_heads=3), "multiple")
    broken(lambda j: j["layers"][0]["mlp"]["router"].update(top=9), "exceeds")
    broken(lambda j: j["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups")
    broken(lambda j: j["norm"].update(groups=5), "norm.groups")
    broken(lambda j: j["layers"][0]["mlp"].update(kind="dense"), "not supported")
    broken(lambda j: j["layers"][0]["mixer"].update(conv="3"), "layers\\[0\\].mixer.conv")


def test_spec_declares_exactly_the_checkpoint_tensors_and_random_mode_lists_them(tmp_path):
    import torch
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.config.registry import get_architecture
    from mlxforge_b200.models.decoder import DecoderModel
    from mlxforge_b200.parts.base import FixedState, PagedKV
    from mlxforge_b200.weights.loader import check_names, tensor_shapes as file_shapes
    from mlxforge_b200.weights.random_init import write_random_model

    class RT:
        dtype, device, precise = torch.float32, torch.device("cpu"), True
    for which, (cfg, ranks) in CONFIGS.items():
        shapes = dict(tensor_shapes(cfg, ranks))
        c = config_from_json(json.loads(json.dumps(cfg))).with_tensor_shapes(shapes)
        arch = get_architecture("Notirax")
        model = DecoderModel(arch.build_spec(c), RT())
        check_names(model.tensor_specs(), shapes)
        assert {n: tuple(s) for n, s, _ in arch.random_tensors(c)} == shapes
        d = write_random_model(str(tmp_path / which), c, seed=3)
        assert file_shapes(d) == shapes
        assert config_from_json(json.load(open(d + "/config.json"))).with_tensor_shapes(file_shapes(d)).to_json() == c.to_json()
    # the cache layout of A: one paged group (two attention lanes with unlike key and value sizes and
    # a chunk), two state groups (the two delta layers differ in size)
    c = config_from_json(json.loads(json.dumps(NX_A))).with_tensor_shapes(dict(tensor_shapes(NX_A, RANKS_A)))
    layout = DecoderModel(get_architecture("Notirax").build_spec(c), RT()).cache_layout
    assert [(g.need, g.n_lanes) for g in layout.paged] == [(PagedKV(1, 8, 0, 7, 16), 2)]
    assert sorted(g.need.shape[0] for g in layout.state) == [2 * 24 * 8 + 1 * (2 * 2 * 24 + 2 * 8),
                                                             4 * 8 * 12 + 3 * (2 * 2 * 8 + 4 * 12)]
    with pytest.raises(ValueError, match="low-rank"):
        get_architecture("Notirax").build_spec(config_from_json(json.loads(json.dumps(NX_A))))


def test_unknown_architecture_lists_the_registered():
    from mlxforge_b200.config import ConfigError, config_from_json
    with pytest.raises(ConfigError, match="LlamaForCausalLM, Luzinex, Notirax"):
        config_from_json({"architecture": "Nothing"})


# ----------------------------------------------------------------------------- cache pages under a chunk mask

def test_chunked_group_gives_pages_back_at_chunk_starts():
    from mlxforge_b200.cache.manager import CacheLayout, CacheManager, GroupLayout
    from mlxforge_b200.parts.base import PagedKV
    import torch
    layout = CacheLayout(paged=(GroupLayout(PagedKV(1, 8, 0, 40, 4), 1), GroupLayout(PagedKV(1, 8), 1)), state=(),
                         item_lane=(("paged", 0, 0), ("paged", 1, 0)))
    cm = CacheManager(layout, page_size=16, max_tokens=256, max_seqs=2, dtype=torch.float32, device="cpu")
    assert cm._v[0].shape[-1] == 4 and cm._k[0].shape[-1] == 8 and cm._v[1].shape[-1] == 8
    seq = cm.open_sequence()
    for n in (30, 9, 1, 1, 45, 2):
        cm.reserve([(seq, n)])
        cm.commit(seq, n)
        cm.check()
        start = seq.length // 40 * 40                   # the chunk of the next query
        first = start // 16
        assert all(p < 0 for p in seq.blocks[0][:first]) and all(p >= 0 for p in seq.blocks[0][first:])
        assert all(p >= 0 for p in seq.blocks[1])
    assert seq.pages_held(0) < seq.pages_held(1)
    cm.close(seq)
    assert cm.free_pages() == cm.total_pages()


# ----------------------------------------------------------------------------- command line without a device

def test_cli_random_weights_and_dump_for_notirax(tmp_path, capsys):
    from mlxforge_b200 import cli
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.weights.loader import tensor_shapes as file_shapes
    cfg = config_from_json(json.loads(json.dumps(NX_A))).with_tensor_shapes(dict(tensor_shapes(NX_A, RANKS_A)))
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(cfg.to_json()))
    out = tmp_path / "model"
    assert cli.main(["random-weights", str(cfg_path), str(out), "--seed", "5"]) == 0
    assert file_shapes(str(out)) == dict(tensor_shapes(NX_A, RANKS_A))
    capsys.readouterr()
    assert cli.main(["dump-weights", str(out)]) == 0
    text = capsys.readouterr().out
    assert "l0.mix.a1 [5, 48] BF16" in text and "l1.mix.talk [4, 4] BF16" in text and "l1.hc1.mix [2, 2] BF16" in text
