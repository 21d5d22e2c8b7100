"""The plain implementation of Luzinex (plain_luzinex.py) against closed forms and against itself
in another form, the configuration reader, the tensor lists and the cache's page discipline under a
window that keeps its first tokens.  No GPU."""
import json

import numpy as np
import pytest

import plain_luzinex as P
from luzinex_helpers import CONFIGS, LZ_A, LZ_B, LZ_C, random_weights, tensor_shapes


def test_rotations_are_rotations_and_agree_up_to_the_pairing():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 2, 12))
    pos = np.array([0, 1, 7, 100, 1000])
    for fn in (P.rotate_half, P.rotate_pairs):
        y = fn(x, pos, 8, 100.0)
        assert np.allclose(y[0], x[0]) and np.allclose(y[..., 8:], x[..., 8:])
        assert np.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    # the pairing is only a permutation of channels: pair i is (i, i + 4) there and (2i, 2i + 1) here
    perm = np.array([0, 4, 1, 5, 2, 6, 3, 7])
    assert np.allclose(P.rotate_pairs(x[..., perm], pos, 8, 100.0), P.rotate_half(x[..., :8], pos, 8, 100.0)[..., perm])
    # relative: a score between rotated vectors depends on the distance only
    q, k = rng.standard_normal((1, 1, 8)), rng.standard_normal((1, 1, 8))
    s = [float((P.rotate_half(q, [p + 5], 8, 50.0) * P.rotate_half(k, [p], 8, 50.0)).sum()) for p in (0, 9, 300)]
    assert np.allclose(s, s[0])
    # pair i turns by position * base^(-2i/dims)
    one = np.zeros((1, 1, 4)); one[0, 0, 1] = 1.0
    y = P.rotate_half(one, [3], 4, 10.0)
    a = 3 * 10.0 ** (-2 * 1 / 4)
    assert np.allclose(y[0, 0], [0, np.cos(a), 0, np.sin(a)])


def test_gelu_and_norm_closed_forms():
    assert abs(P.gelu_tanh(np.array(1.0)) - 0.8411919906082768) < 1e-12
    assert P.gelu_tanh(np.array(0.0)) == 0.0 and abs(P.gelu_tanh(np.array(-10.0))) < 1e-12
    x = np.array([[3.0, 4.0]])
    assert np.allclose(P.rms_norm(x, np.array([2.0, 1.0]), 0.0), [[2 * 3 / np.sqrt(12.5), 4 / np.sqrt(12.5)]])
    assert np.allclose(P.rms_norm(np.zeros((1, 4)), None, 1e-5), 0.0)


def test_mask_window_and_kept_first_tokens():
    m = P.visible(12, window=4, keep_first=2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert m[3].tolist() == [True] * 4 + [False] * 8 and m[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert (P.visible(5) == np.tril(np.ones((5, 5), bool))).all()
    assert (P.visible(9, window=3, keep_first=0)[8] == np.array([0, 0, 0, 0, 0, 0, 1, 1, 1], bool)).all()


def test_sink_is_one_more_term_of_the_denominator():
    s = np.log(np.array([[[1.0, 3.0]]]))          # one head, one query, two keys
    w = P.masked_softmax(s, np.ones((1, 2), bool), np.array([np.log(4.0)]))
    assert np.allclose(w, [[[1 / 8, 3 / 8]]])
    w = P.masked_softmax(s, np.ones((1, 2), bool), np.array([-np.inf]))
    assert np.allclose(w, [[[1 / 4, 3 / 4]]])


def test_latent_attention_equals_attention_over_the_latent():
    """The form the engine computes: queries mapped into the latent, keys the cached rows themselves."""
    rng = np.random.default_rng(3)
    m = LZ_A["layers"][0]["mixer"]
    H, T = 48, 9
    w = {k[len("l0.mix."):]: v.astype(np.float64) for k, v in random_weights(LZ_A, 1).items() if k.startswith("l0.mix.")}
    h = rng.standard_normal((T, H))
    want, (c, kr) = P.latent_attention(h, w, m, 1e-5)
    nh, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = P.rms_norm(h @ w["dq"].T, w["dq.norm"], 1e-5)
    q = (cq @ w["uq"].T).reshape(T, nh, d + r)
    qa = np.einsum("thd,hdr->thr", q[..., :d], w["uk"].reshape(nh, d, rank))
    qr = P.rotate_half(q[..., d:], np.arange(T), r, m["rot"]["base"])
    s = (np.einsum("ihr,jr->hij", qa, c) + np.einsum("ihr,jr->hij", qr, kr)) * m["scale"]
    p = P.masked_softmax(s, P.visible(T))
    o = np.einsum("hij,jr->ihr", p, c)
    o = np.einsum("ihr,hvr->ihv", o, w["uv"].reshape(nh, dv, rank)).reshape(T, nh * dv) * P.sigmoid(h @ w["g"].T)
    assert np.allclose(o @ w["o"].T, want, atol=1e-10)


def test_retention_first_token_full_decay_and_sum_form():
    rng = np.random.default_rng(5)
    m = {"heads": 2, "dim": 4, "vdim": 3, "decay": [0.0, 1.0], "rot": {"base": 10.0, "dims": 4}}
    H, T = 6, 7
    w = {n: rng.standard_normal(s) for n, s in (("q", (8, H)), ("k", (8, H)), ("v", (6, H)), ("g", (6, H)), ("o", (H, 6)))}
    h = rng.standard_normal((T, H))
    out, S = P.retention(h, w, m, 1e-5)
    pos = np.arange(T)
    q = P.rotate_half((h @ w["q"].T).reshape(T, 2, 4), pos, 4, 10.0)
    k = P.rotate_half((h @ w["k"].T).reshape(T, 2, 4), pos, 4, 10.0) * 0.5
    v = (h @ w["v"].T).reshape(T, 2, 3)
    # decay 0: only the token itself; decay 1: the plain sum over the past
    o0 = np.einsum("td,td->t", q[:, 0], k[:, 0])[:, None] * v[:, 0]
    o1 = np.stack([sum((q[t, 1] @ k[j, 1]) * v[j, 1] for j in range(t + 1)) for t in range(T)])
    o = np.stack([o0, o1], axis=1)
    want = (P.rms_norm(o, None, 1e-5).reshape(T, 6) * P.silu(h @ w["g"].T)) @ w["o"].T
    assert np.allclose(out, want, atol=1e-10)
    # the state carries on: two halves equal the whole
    a, Sa = P.retention(h[:3], w, m, 1e-5)
    m2 = dict(m)
    assert np.allclose(Sa[1], sum(np.outer(k[j, 1], v[j, 1]) for j in range(3)))


def test_whole_model_runs_and_layers_are_reported():
    for which, cfg in CONFIGS.items():
        w = {k: v.astype(np.float64) for k, v in random_weights(cfg, 2).items()}
        layers = []
        logits = P.forward(cfg, w, [1, 5, 3, 0, 7, 7, 2], layers)
        assert logits.shape == (7, cfg["vocab"]) and len(layers) == len(cfg["layers"]) and np.isfinite(logits).all()
        # causal: a prefix gives the same logits
        assert np.allclose(P.forward(cfg, w, [1, 5, 3, 0])[:4], logits[:4], atol=1e-9)


# ----------------------------------------------------------------------------- configuration and tensors

def test_configuration_reader_defaults_errors_and_round_trip():
    from mlxforge_b200.config import ConfigError, config_from_json
    from mlxforge_b200.config.registry import get_architecture
    for cfg in (LZ_A, LZ_B, LZ_C):
        c = config_from_json(json.loads(json.dumps(cfg)))
        assert c.architecture == "Luzinex" and len(c.layers) == len(cfg["layers"])
        assert config_from_json(c.to_json()).layers == c.layers
        arch = get_architecture("Luzinex")
        assert [(n, tuple(s)) for n, s, _ in arch.random_tensors(c)] == [(n, tuple(s)) for n, s in tensor_shapes(cfg)]
        spec = arch.build_spec(c)
        for i, layer in enumerate(cfg["layers"]):
            assert spec.schedule[i].cache_of == layer["mixer"].get("kv_from")
            assert (spec.layers[i].feed_forward is None) == (layer["mlp"] is None)
    c = config_from_json(json.loads(json.dumps(LZ_B)))
    assert c.layers[0]["mixer"]["window"] == 0 and c.layers[3]["mixer"]["keep_first"] == 0

    def broken(path, value):
        j = json.loads(json.dumps(LZ_A))
        o = j
        for k in path[:-1]:
            o = o[k]
        if value is None:
            del o[path[-1]]
        else:
            o[path[-1]] = value
        return j
    for path, value, text in [(("width",), None, "'width'"), (("norm", "eps"), None, "'norm.eps'"),
                              (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
                              (("layers", 0, "type"), "conv", "not supported"),
                              (("layers", 0, "mlp", "kind"), "moe", "not supported"),
                              (("layers", 2, "mixer", "decay"), [0.5], "one number per head"),
                              (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 1, "mixer", "vdim"), 8, "values of this mixer are its keys"),
                              (("layers", 3, "mixer", "kv_from"), 1, "kv_from"),
                              (("layers", 3, "mixer", "kv_from"), 3, "kv_from"),
                              (("layers", 3, "mixer", "kv_rank"), 16, "kv_from"),
                              (("layers", 1, "mixer", "heads"), 3, "multiple")]:
        with pytest.raises(ConfigError, match=text):
            config_from_json(broken(path, value))


def test_cache_layout_shares_the_latent_lane_and_keeps_the_first_pages():
    from mlxforge_b200.cache.manager import CacheManager
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.config.registry import get_architecture
    from mlxforge_b200.models.decoder import DecoderModel
    from mlxforge_b200.parts.base import PagedKV

    class RT:
        dtype = None
        precise = True
        device = "cpu"

        def buffer(self, *a, **k):
            raise AssertionError("no scratch at build time")
    import torch
    RT.dtype = torch.float32
    c = config_from_json(json.loads(json.dumps(LZ_A)))
    model = DecoderModel(get_architecture("Luzinex").build_spec(c), RT())
    layout = model.cache_layout
    needs = [(g.need, g.n_lanes) for g in layout.paged]
    assert (PagedKV(1, 28, v_head_dim=24, values_in_keys=True), 1) in needs           # layer 3 adds no lane
    assert (PagedKV(2, 24, 11, keep_first=3), 1) in needs and (PagedKV(1, 16, 37, keep_first=17), 1) in needs
    assert layout.item_lane[3] == layout.item_lane[0]
    assert [g.need.shape for g in layout.state] == [(3 * 12 * 20,)]
    # pages under a window of 37 that keeps 17 tokens (two pages of 16): blocks 0 and 1 stay for ever
    cache = CacheManager(layout, page_size=16, max_tokens=64 * 4, max_seqs=2, dtype=torch.float32, device="cpu")
    g = [i for i, gl in enumerate(layout.paged) if gl.need.window == 37][0]
    seq = cache.open_sequence()
    for n in (50, 1, 1, 30, 1, 40):
        cache.reserve([(seq, n)])
        cache.commit(seq, n)
        first = max(0, seq.length - 37 + 1) // 16
        held = [b for b, p in enumerate(seq.blocks[g]) if p >= 0]
        assert held == sorted(set([0, 1][:len(seq.blocks[g])]) | set(range(first, len(seq.blocks[g])))), (seq.length, held)
        cache.check()
    cache.close(seq)
    assert cache.free_pages() == cache.total_pages()
