"""The Luzinex parts and models on the GPU against the plain implementation (plain_luzinex.py).

Mechanism by mechanism (each part built from its registry with its own sizes, given a runtime, a
step batch and a cache lane, run over portions and single tokens of two sequences with pools full
of NaN), edge keys made to decide, then whole models of three configurations through the trace
replayer's functions -- whole prompts, the last tokens decoded one by one, portions down to two
tokens, mixed batches on a pool so small that pages and slots are used again, every request decoded
from its first token -- in float32 and bfloat16, and greedy generation through the engine's entry
point and scheduler."""
import io

import numpy as np
import pytest

import plain_luzinex as P
import trace_tools as TT
from luzinex_helpers import CONFIGS, make_model, prompt
from test_notirax_gpu import Harness, dev, host, rand, tdt, tol

pytestmark = pytest.mark.gpu

LONG = [150, 70]
LONG_STEPS = [(90, 0), (40, 33), (1, 30), (17, 1), (1, 1), (1, 5)]


def spec(kind, params, prefix="m."):
    from mlxforge_b200.parts.base import PartSpec
    return PartSpec(kind, params, prefix)


def build(registry, kind, params, rt, tensors, prefix="m."):
    from mlxforge_b200.parts import base
    part = base.build_part(getattr(base, registry), spec(kind, params, prefix), rt)
    specs = part.tensor_specs()
    assert set(specs) == set(tensors), (sorted(specs), sorted(tensors))
    for n, s in specs.items():
        assert tuple(s.shape) == tuple(tensors[n].shape), (n, s.shape, tensors[n].shape)
    part.bind({n: dev(a) for n, a in tensors.items()})
    return part


# ----------------------------------------------------------------------------- norm pair, feed-forward

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H", [40, 33, 256, 2048])
def test_add_and_two_norms_of_one_sum(dtype, H):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(H)
    T, eps = 6, 1e-5
    x = rng.standard_normal((T, H)).astype(np.float32) * 3
    d1, d2 = rand(rng, T, H), rand(rng, T, H)
    w1, w2 = (1 + 0.2 * rng.standard_normal((2, H))).astype(np.float32)
    f = np.float64
    for a, b in ((d1, d2), (d1, None), (None, d2), (None, None)):
        s = x.astype(f) + (0 if a is None else a) + (0 if b is None else b)
        resid = dev(x)
        o1 = torch.empty((T, H), dtype=tdt(dtype), device="cuda")
        o2 = torch.empty((T, H), dtype=tdt(dtype), device="cuda")
        ops.add_rmsnorm_pair(resid, None if a is None else dev(a, tdt(dtype)), None if b is None else dev(b, tdt(dtype)),
                             dev(w1), dev(w2), eps, o1, o2)
        assert np.max(np.abs(host(o1) - P.rms_norm(s, w1.astype(f), eps))) < tol(dtype, 4.0)
        assert np.max(np.abs(host(o2) - P.rms_norm(s, w2.astype(f), eps))) < tol(dtype, 4.0)
        assert np.max(np.abs(host(resid) - s)) < 1e-5
    # selected rows: the residual stays, one norm only
    resid = dev(x)
    rows = dev(np.array([4, 0, 4], dtype=np.int32))
    o1 = torch.empty((3, H), dtype=tdt(dtype), device="cuda")
    ops.add_rmsnorm_pair(resid, dev(d1, tdt(dtype)), dev(d2, tdt(dtype)), dev(w1), None, eps, o1, None, rows)
    s = x.astype(f) + d1 + d2
    assert np.max(np.abs(host(o1) - P.rms_norm(s, w1.astype(f), eps)[[4, 0, 4]])) < tol(dtype, 4.0)
    assert np.array_equal(host(resid), x.astype(f))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,ff,T", [(40, 20, 5), (64, 72, 3), (256, 512, 300), (128, 96, 40)])
def test_gelu_gated_feed_forward(dtype, H, ff, T):
    from mlxforge_b200.engine.runtime import Runtime
    rng = np.random.default_rng(ff)
    rt = Runtime(tdt(dtype))
    w = {"m.gate": rand(rng, ff, H, std=H ** -0.5), "m.up": rand(rng, ff, H, std=H ** -0.5),
         "m.down": rand(rng, H, ff, std=ff ** -0.5)}
    part = build("FEED_FORWARDS", "swiglu", {"hidden_size": H, "intermediate_size": ff, "activation": "gelu_tanh",
                                             "names": {"gate": "gate", "up": "up", "down": "down"}}, rt, w)
    x = rand(rng, T, H, std=2.0)
    want = P.gelu_ff(x.astype(np.float64), *(w[k].astype(np.float64) for k in ("m.gate", "m.up", "m.down")))
    got = host(part.forward(dev(x, tdt(dtype)), None))
    assert np.max(np.abs(got - want)) < tol(dtype, np.abs(want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,heads,N,K,gated", [(5, 3, 7, 12, True), (1, 1, 40, 16, False), (150, 4, 48, 32, True),
                                               (70, 2, 100, 64, True), (300, 6, 64, 48, False), (33, 2, 24, 20, True)])
def test_a_product_per_head(dtype, T, heads, N, K, gated):
    """Rows and heads of x and of the result sit inside wider rows (other columns must stay as they are); few
    tokens and sizes the tensor-core kernel does not take go through the kernel with a warp per output."""
    import torch
    from mlxforge_b200.csrc import binding
    from mlxforge_b200.engine.runtime import Runtime
    rng = np.random.default_rng(T + N)
    rt = Runtime(tdt(dtype))
    x_hs, out_hs = K + 8, N + 3
    x_ld, out_ld = heads * x_hs + 16, heads * out_hs + 5
    x = rand(rng, T, x_ld)
    w = rand(rng, heads, N, K, std=K ** -0.5)
    gate = rand(rng, T, heads * N + 6)
    out = torch.full((T, out_ld), 7.0, dtype=tdt(dtype), device="cuda")
    xd, gd = dev(x, tdt(dtype)), dev(gate, tdt(dtype))
    before = binding.kernel_launches()
    rt.head_linear(xd[:, 8:], x_ld, x_hs, dev(w, tdt(dtype)), out[:, 2:], out_ld, out_hs, T,
                   gd[:, 6:] if gated else None, gate.shape[1])
    ran = {k: v - before[k] for k, v in binding.kernel_launches().items() if v - before[k]}
    want = np.full((T, out_ld), 7.0)
    for h in range(heads):
        y = x[:, 8 + h * x_hs:8 + h * x_hs + K].astype(np.float64) @ w[h].astype(np.float64).T
        if gated:
            y = y * P.sigmoid(gate[:, 6 + h * N:6 + (h + 1) * N].astype(np.float64))
        want[:, 2 + h * out_hs:2 + h * out_hs + N] = y
    assert np.max(np.abs(host(out) - want)) < tol(dtype, 4.0)
    tensor_cores = dtype == "bfloat16" and T > 16 and K % 16 == 0
    assert ("head_linear_mma" in ran) == tensor_cores and ("head_linear" in ran) != tensor_cores, ran


# ----------------------------------------------------------------------------- the attention whose values are its keys

SINK_CASES = {
    # heads, kv heads, dim, rotated dims, window, kept, pairing
    "odd": (4, 2, 24, 8, 11, 3, "pairs"),
    "no_mask": (2, 2, 16, 16, 0, 0, "pairs"),
    "page_window": (3, 1, 16, 2, 16, 0, "half"),
    "kept_pages": (2, 1, 32, 32, 21, 35, "pairs"),
    "tc64": (4, 2, 64, 32, 40, 5, "pairs"),
    "tc128": (2, 1, 128, 64, 70, 17, "pairs"),
}


def sink_part(case, dtype, rt, rng, H=40, gain=1.0):
    nh, nkv, d, rot, window, keep, pairing = SINK_CASES[case]
    w = {"m.q": rand(rng, nh * d, H, std=gain * H ** -0.5), "m.k": rand(rng, nkv * d, H, std=gain * H ** -0.5),
         "m.g": rand(rng, nh * d, H, std=H ** -0.5), "m.o": rand(rng, H, nh * d, std=(nh * d) ** -0.5),
         "m.sink": rand(rng, nh)}
    params = {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d, "softmax_scale": 0.3, "window": window,
              "keep_first": keep, "values": "keys", "sink": True, "gate": True,
              "position": spec("rotary", {"head_dim": d, "rotary_dim": rot, "base": 300.0, "pairing": pairing}, "")}
    m = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": d, "scale": 0.3, "rot": {"base": 300.0, "dims": rot},
         "mask": {"size": window, "keep_first": keep} if window else None}
    return build("MIXERS", "sink_attention", params, rt, w), w, m


def plain_sink(x, w, m, pairing="pairs"):
    p = {k[2:]: v.astype(np.float64) for k, v in w.items()}
    if pairing == "half":      # the plain function rotates pairs (2i, 2i+1): permute q's and k's channels so that it does
        d, r = m["dim"], m["rot"]["dims"]
        perm = np.arange(d)
        perm[:r] = np.concatenate([[i, i + r // 2] for i in range(r // 2)])
        for n in ("q", "k"):
            a = p[n].reshape(-1, d, p[n].shape[1])
            p[n] = a[:, perm].reshape(p[n].shape)
        # values are the keys and the output follows their channel order: undo it behind the attention
        inv = np.argsort(perm)
        nh = m["heads"]
        p["g"] = p["g"].reshape(nh, d, -1)[:, perm].reshape(p["g"].shape)
        p["o"] = p["o"].reshape(-1, nh, d)[:, :, perm].reshape(p["o"].shape)
    return P.sink_window_attention(x.astype(np.float64), p, m)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(SINK_CASES))
def test_sink_attention_part(dtype, case):
    from mlxforge_b200.csrc import binding
    rng = np.random.default_rng(len(case))
    big = case.startswith("tc") or case == "kept_pages"
    from mlxforge_b200.parts.base import PagedKV
    nh, nkv, d, rot, window, keep, pairing = SINK_CASES[case]
    h = Harness(dtype, PagedKV(nkv, d, window, keep_first=keep if window else 0), lengths=LONG if big else [45, 23],
                steps=LONG_STEPS if big else [(20, 0), (7, 5), (0, 16), (17, 1), (1, 1)])
    part, w, m = sink_part(case, dtype, h.rt, rng)
    assert part.cache_need() == h.cache.layout.paged[0].need
    xs = [rand(rng, n, 40) for n in h.lengths]
    before = binding.kernel_launches()
    got = h.run_mixer(part, xs, dtype)
    ran = {k: v - before[k] for k, v in binding.kernel_launches().items() if v - before[k]}
    for x, g in zip(xs, got):
        want = plain_sink(x, w, m, SINK_CASES[case][6])
        assert np.max(np.abs(g - want)) < tol(dtype, np.abs(want).max()), (case, np.max(np.abs(g - want)))
    if dtype == "bfloat16" and case.startswith("tc"):
        assert ran.get("attn_prefill_mma", 0) > 0 and ran.get("attn_decode", 0) > 0 and "attn_generic" not in ran, ran


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["odd", "kept_pages", "tc64", "tc128"])
def test_keys_at_the_edges_of_the_window_and_of_the_kept_tokens_decide(dtype, case):
    """Scores come from one unrotated channel alone: every query has 1 there, a key what its token says.  The
    keys just inside and just outside the window of the last queries, the last kept token and the first one
    that is not kept, and keys on both sides of page borders get a large entry each, so that one key too
    many or too few changes the output by a large factor."""
    from mlxforge_b200.parts.base import PagedKV
    nh, nkv, d, rot, window, keep, pairing = SINK_CASES[case]
    rot = min(rot, d - 2)                       # leave a channel that does not rotate
    H, n = 8, 150
    rng = np.random.default_rng(7)
    c = d - 1                                   # the unrotated channel
    wq, wk = np.zeros((nh * d, H), np.float32), np.zeros((nkv * d, H), np.float32)
    for hh in range(nh):
        wq[hh * d + c, 0] = 1.0
    for g in range(nkv):
        wk[g * d + c, 1] = 1.0
        wk[g * d:(g + 1) * d - 1, 2:] = rng.standard_normal((d - 1, H - 2)) * 1.5      # what the values carry
    w = {"m.q": wq, "m.k": wk, "m.g": np.zeros((nh * d, H), np.float32),
         "m.o": rand(rng, H, nh * d, std=0.2), "m.sink": np.zeros(nh, np.float32)}
    params = {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d, "softmax_scale": 1.0, "window": window,
              "keep_first": keep, "values": "keys", "sink": True, "gate": True,
              "position": spec("rotary", {"head_dim": d, "rotary_dim": rot, "base": 300.0, "pairing": "pairs"}, "")}
    m = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": d, "scale": 1.0, "rot": {"base": 300.0, "dims": rot},
         "mask": {"size": window, "keep_first": keep}}
    x = rand(rng, n, H, std=0.5)
    x[:, 0], x[:, 1] = 1.0, 0.0
    last = n - 1
    marked = {last - window, last - window + 1, last - window - 1, keep - 1, keep, 15, 16, 31, 32,
              (last - 20) - window, (last - 20) - window + 1, last}
    for j in marked:
        if 0 <= j < n:
            x[j, 1] = 12.0
    h = Harness(dtype, PagedKV(nkv, d, window, keep_first=keep), lengths=[n], steps=[(100,), (29,)] + [(1,)] * 21)
    part = build("MIXERS", "sink_attention", params, h.rt, w)
    got = h.run_mixer(part, [x], dtype)[0]
    want = P.sink_window_attention(x.astype(np.float64), {k[2:]: v.astype(np.float64) for k, v in w.items()}, m)
    # the check has teeth: a window one longer or one kept token more gives another answer at the last queries
    for wrong in ({"size": window + 1, "keep_first": keep}, {"size": window, "keep_first": keep + 1},
                  {"size": window - 1, "keep_first": keep}):
        other = P.sink_window_attention(x.astype(np.float64), {k[2:]: v.astype(np.float64) for k, v in w.items()},
                                        dict(m, mask=wrong))
        assert np.max(np.abs(other[-22:] - want[-22:])) > 1.5 * tol(dtype, np.abs(want).max())
    assert np.max(np.abs(got - want)) < tol(dtype, np.abs(want).max()), np.argmax(np.abs(got - want).max(axis=1))


# ----------------------------------------------------------------------------- attention over the latent

LATENT_CASES = {
    # heads, dim, rot, vdim, q_rank, kv_rank
    "odd": (3, 8, 4, 12, 20, 24),
    "ones": (1, 16, 2, 16, 8, 6),
    "tc64": (4, 32, 16, 32, 64, 48),
    "tc96": (6, 16, 32, 48, 40, 64),
    "wide": (2, 24, 8, 16, 32, 280),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(LATENT_CASES))
def test_latent_attention_part(dtype, case):
    from mlxforge_b200.csrc import binding
    from mlxforge_b200.parts.base import PagedKV
    nh, d, rot, dv, qr, kr = LATENT_CASES[case]
    H = 40
    rng = np.random.default_rng(len(case) + nh)
    w = {"m.dq": rand(rng, qr, H, std=H ** -0.5), "m.dq.norm": 1 + 0.1 * rand(rng, qr),
         "m.uq": rand(rng, nh * (d + rot), qr, std=2 * qr ** -0.5), "m.dkv": rand(rng, kr + rot, H, std=H ** -0.5),
         "m.dkv.norm": 1 + 0.1 * rand(rng, kr), "m.uk": rand(rng, nh * d, kr, std=2 * kr ** -0.5),
         "m.uv": rand(rng, nh * dv, kr, std=kr ** -0.5), "m.g": rand(rng, nh * dv, H, std=H ** -0.5),
         "m.o": rand(rng, H, nh * dv, std=(nh * dv) ** -0.5)}
    w = {k: np.asarray(v, np.float32) for k, v in w.items()}
    big = case.startswith("tc")
    h = Harness(dtype, PagedKV(1, kr + rot, v_head_dim=kr, values_in_keys=True), lengths=LONG if big else [45, 23],
                steps=LONG_STEPS if big else [(20, 0), (7, 5), (0, 16), (17, 1), (1, 1)])
    params = {"hidden_size": H, "n_heads": nh, "head_dim": d, "rot_dim": rot, "v_head_dim": dv, "q_rank": qr,
              "kv_rank": kr, "softmax_scale": 0.4, "rope_base": 777.0, "eps": 1e-5, "gate": True}
    part = build("MIXERS", "latent_attention", params, h.rt, w)
    assert part.cache_need() == h.cache.layout.paged[0].need
    assert h.cache.lane(0).v.data_ptr() == h.cache.lane(0).k.data_ptr()          # no value pool of its own
    m = {"heads": nh, "dim": d, "rot_dim": rot, "vdim": dv, "kv_rank": kr, "scale": 0.4, "rot": {"base": 777.0}}
    xs = [rand(rng, n, H) for n in h.lengths]
    before = binding.kernel_launches()
    got = h.run_mixer(part, xs, dtype)
    ran = {k: v - before[k] for k, v in binding.kernel_launches().items() if v - before[k]}
    for x, g in zip(xs, got):
        want, _ = P.latent_attention(x.astype(np.float64), {k[2:]: v.astype(np.float64) for k, v in w.items()}, m, 1e-5)
        assert np.max(np.abs(g - want)) < tol(dtype, np.abs(want).max()), (case, np.max(np.abs(g - want)))
    assert ran.get("latent_prepare", 0) > 0
    if dtype == "bfloat16" and big:
        assert ran.get("attn_prefill_mma", 0) > 0 and ran.get("attn_decode", 0) > 0 and "attn_generic" not in ran, ran


# ----------------------------------------------------------------------------- retention

RET_CASES = {
    # heads, dim, vdim, rotated dims, decays
    "odd": (3, 12, 20, 8, (0.9, 0.99, 0.75)),
    "ones": (1, 16, 16, 16, (1.0,)),
    "d64": (2, 64, 32, 64, (0.97, 0.9995)),
    "d128": (2, 128, 64, 32, (0.5, 0.999)),
    "d200": (1, 200, 24, 0, (0.98,)),
    "d320": (1, 320, 8, 320, (0.9,)),
}


def ret_part(case, rt, rng, H=40):
    nh, d, dv, rot, decay = RET_CASES[case]
    w = {"m.q": rand(rng, nh * d, H, std=H ** -0.5), "m.k": rand(rng, nh * d, H, std=H ** -0.5),
         "m.v": rand(rng, nh * dv, H, std=H ** -0.5), "m.g": rand(rng, nh * dv, H, std=H ** -0.5),
         "m.o": rand(rng, H, nh * dv, std=(nh * dv) ** -0.5)}
    params = {"hidden_size": H, "n_heads": nh, "head_dim": d, "v_head_dim": dv, "rotary_dim": rot, "rope_base": 5000.0,
              "decay": decay, "eps": 1e-5}
    m = {"heads": nh, "dim": d, "vdim": dv, "decay": list(decay), "rot": {"base": 5000.0, "dims": rot}}
    return build("MIXERS", "retention", params, rt, w), w, m


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(RET_CASES))
def test_retention_part(dtype, case):
    from mlxforge_b200.parts.base import FixedState
    nh, d, dv, rot, decay = RET_CASES[case]
    rng = np.random.default_rng(d)
    big = d >= 64
    h = Harness(dtype, FixedState((nh * d * dv,), tag="retention"), lengths=LONG if big else [45, 23],
                steps=LONG_STEPS if big else [(20, 0), (7, 5), (0, 16), (17, 1), (1, 1)])
    part, w, m = ret_part(case, h.rt, rng)
    assert part.cache_need() == h.cache.layout.state[0].need
    xs = [rand(rng, n, 40) for n in h.lengths]
    got = h.run_mixer(part, xs, dtype)
    for x, g in zip(xs, got):
        want, _ = P.retention(x.astype(np.float64), {k[2:]: v.astype(np.float64) for k, v in w.items()}, m, 1e-5)
        assert np.max(np.abs(g - want)) < tol(dtype, np.abs(want).max()), (case, np.max(np.abs(g - want)))


def test_retention_state_carries_a_far_token():
    """A head that never forgets (decay 1): one early token with a large key and value, then hundreds of small
    ones, token by token; the last read-out is that early token's value only if the state is intact."""
    from mlxforge_b200.parts.base import FixedState
    nh, d, dv, H, n = 1, 16, 16, 8, 400
    rng = np.random.default_rng(1)
    w = {"m.q": np.zeros((d, H), np.float32), "m.k": np.zeros((d, H), np.float32), "m.v": rand(rng, dv, H, std=1.0),
         "m.g": np.zeros((dv, H), np.float32), "m.o": rand(rng, H, dv, std=0.3)}
    w["m.q"][d - 1, 0] = 1.0
    w["m.k"][d - 1, 1] = 1.0
    w["m.g"][:, 0] = 2.0
    params = {"hidden_size": H, "n_heads": nh, "head_dim": d, "v_head_dim": dv, "rotary_dim": d - 2, "rope_base": 100.0,
              "decay": (1.0,), "eps": 1e-6}
    m = {"heads": nh, "dim": d, "vdim": dv, "decay": [1.0], "rot": {"base": 100.0, "dims": d - 2}}
    x = rand(rng, n, H, std=0.3)
    x[:, 0], x[:, 1] = 1.0, 0.001
    x[3, 1] = 50.0
    steps = [(2,), (3,), (150,)] + [(1,)] * 245
    h = Harness("float32", FixedState((nh * d * dv,), tag="retention"), lengths=[n], steps=steps)
    part = build("MIXERS", "retention", params, h.rt, w)
    got = h.run_mixer(part, [x], "float32")[0]
    want, _ = P.retention(x.astype(np.float64), {k[2:]: v.astype(np.float64) for k, v in w.items()}, m, 1e-6)
    x2 = x.copy()
    x2[3, 1] = 0.001
    without, _ = P.retention(x2.astype(np.float64), {k[2:]: v.astype(np.float64) for k, v in w.items()}, m, 1e-6)
    assert np.max(np.abs(without[-1] - want[-1])) > 0.1 * np.abs(want[-1]).max()
    assert np.max(np.abs(got - want)) < 1e-4 * np.abs(want).max()


# ----------------------------------------------------------------------------- whole models

REQUEST_LENGTHS = {"A": [45, 23, 1, 60, 37, 2], "B": [40, 18, 33, 1], "C": [300, 150, 1, 260, 90]}
PORTIONS = {"A": (7, 2, 5, 3, 2, 11, 4, 2, 16, 1, 9), "B": (2, 3, 16, 2, 1, 17), "C": (130, 2, 64, 3, 70, 1, 16)}
PEAKED = {"A": 5.0, "B": 5.0, "C": 3.0}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("luzinex")
    out = {}
    for which in CONFIGS:
        for peaked in (False, True):
            d, cfg, w = make_model(tmp, which, seed=ord(which), qk_gain=PEAKED[which] if peaked else 1.0)
            reqs = {f"r{i}": prompt(cfg, n, i) for i, n in enumerate(REQUEST_LENGTHS[which])}
            expected = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
            noise, loose = _bf16_noise(cfg, w, reqs, expected)
            scale = max(float(np.max(np.abs(e))) for e in expected.values())
            out[(which, peaked)] = (d, cfg, reqs, expected,
                                    {"float32": 1e-4 * max(1.0, scale), "bfloat16": 3.0 * noise, "loose": loose}, w)
    return out


def _bf16_noise(cfg, w, reqs, expected):
    """How far rounding alone moves the logits: the plain implementation with every activation rounded to
    bfloat16 where the engine rounds, and three more times with the rounding dithered by one unit in the last
    place.  The first gives the tolerance of the model; the others say at which positions the model itself is
    ill-conditioned (a retention read-out that is nearly zero before it is normalised flips its sign with the
    last bit of a key), and those positions get a tolerance of their own."""
    rng = np.random.default_rng(0)
    loose = {}
    try:
        P.ROUND = P.round_bf16
        noise = max(float(np.max(np.abs(P.forward(cfg, w, toks) - expected[rid]))) for rid, toks in reqs.items())
        for _ in range(3):
            P.ROUND = lambda x: P.round_bf16(np.asarray(x) * (1.0 + rng.uniform(-1, 1, np.shape(x)) * 2.0 ** -8))
            for rid, toks in reqs.items():
                d = np.max(np.abs(P.forward(cfg, w, toks) - expected[rid]), axis=-1)
                loose[rid] = np.maximum(loose.get(rid, 0.0), d)
    finally:
        P.ROUND = None
    return noise, loose


def _replay(model_dir, dtype, trace, tmp_path, max_tokens=None, max_seqs=4):
    from mlxforge_b200.csrc import binding
    from mlxforge_b200.engine.replay import make_runner, replay
    runner = make_runner(model_dir, dtype, max_tokens or trace.live_tokens_rounded(), max_seqs=max_seqs)
    for pool in runner.cache._k + runner.cache._v + runner.cache._state:
        pool.fill_(float("nan"))
    out_dir = str(tmp_path / "out")
    before = binding.kernel_launches()
    replay(runner, trace.lines(), out_dir, done=io.StringIO())
    runner.cache.check()
    assert runner.cache.free_pages() == runner.cache.total_pages() and runner.cache.slots.n_free == max_seqs
    ran = {k: v - before[k] for k, v in binding.kernel_launches().items() if v - before[k]}
    return out_dir, ran


def _check(models, which, peaked, dtype, trace, tmp_path, **kw):
    d, cfg, reqs, expected, tols, _ = models[(which, peaked)]
    out_dir, ran = _replay(d, dtype, trace, tmp_path, **kw)
    got = TT.read_outputs(trace, out_dir, cfg["vocab"])
    assert got, "the trace asked for nothing"
    bad = []
    for (rid, pos), row in got.items():
        diff = float(np.max(np.abs(row.astype(np.float64) - expected[rid][pos])))
        limit = tols[dtype] if dtype == "float32" else max(tols[dtype], 4.0 * float(tols["loose"][rid][pos]))
        if not diff <= limit:
            bad.append((pos, rid, diff, limit))
    assert not bad, (which, peaked, dtype, len(bad), sorted(bad)[:4])
    return ran


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_residual_stream_after_every_layer(models, dtype):
    from mlxforge_b200.engine.replay import make_runner
    from mlxforge_b200.engine.step import StepEntry
    d, cfg, reqs, _, _, w = models[("A", False)]
    layers, rounded = [], []
    P.forward(cfg, w, reqs["r0"], layers)
    P.ROUND = P.round_bf16
    try:
        P.forward(cfg, w, reqs["r0"], rounded)
    finally:
        P.ROUND = None
    runner = make_runner(d, dtype, 64)
    got = []

    def probe(i, resid, pending):
        x = resid.clone()
        for delta in (pending.first, pending.second):
            if delta is not None:
                x += delta.float()
        got.append(host(x))
    runner.model.probe = probe
    seq = runner.cache.open_sequence()
    runner.step([StepEntry(seq, reqs["r0"], [0])])
    assert len(got) == len(layers)
    for i, (g, want) in enumerate(zip(got, layers)):
        limit = 1e-5 * np.abs(want).max() if dtype == "float32" else 4.0 * np.max(np.abs(rounded[i] - want))
        assert np.max(np.abs(g - want)) < limit, (i, cfg["layers"][i]["type"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("peaked", [False, True])
@pytest.mark.parametrize("which", list(CONFIGS))
def test_whole_prompts_and_decoded_tails(models, which, peaked, dtype, tmp_path):
    reqs = models[(which, peaked)][2]
    _check(models, which, peaked, dtype, TT.whole(reqs), tmp_path)
    _check(models, which, peaked, dtype, TT.decode_tail(reqs, tail=40), tmp_path / "tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(CONFIGS))
def test_portions_down_to_two_tokens(models, which, dtype, tmp_path):
    reqs = models[(which, True)][2]
    _check(models, which, True, dtype, TT.portions(reqs, PORTIONS[which]), tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(CONFIGS))
def test_mixed_batches_on_a_pool_where_pages_and_slots_are_used_again(models, which, dtype, tmp_path):
    reqs = models[(which, True)][2]
    trace = TT.mixed(reqs, max_live=3, seed=3, decode_last=6, max_portion=9 if which != "C" else 140)
    assert trace.live_tokens_rounded() < sum((len(t) + 63) // 64 * 64 for t in reqs.values())
    _check(models, which, True, dtype, trace, tmp_path, max_seqs=3)
    # each request alone gives what it gave inside the batch: the tolerance above holds for both


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_every_request_decoded_from_its_first_token(models, which, dtype, tmp_path):
    """Long decoding (300 steps for C) in a batch that shrinks: the first tokens of a sequence, window edges, kept
    tokens, page borders and the decode kernel's splits met token by token, decode steps replayed from graphs."""
    reqs = models[(which, False)][2]
    _check(models, which, False, dtype, TT.lockstep(reqs), tmp_path, max_seqs=len(reqs))


def test_serving_shapes_take_the_fast_kernels(models, tmp_path):
    """Configuration C in bfloat16: which kernels its prompts and its decoding go through."""
    reqs = models[("C", False)][2]
    ran = _check(models, "C", False, "bfloat16", TT.decode_tail(reqs, tail=8), tmp_path)
    for k in ("norm_pair", "rope_store", "latent_prepare", "latent_query", "head_linear", "head_linear_mma", "retention_prepare",
              "retention_recurrence", "retention_output", "attn_prefill_mma", "attn_decode", "attn_decode_merge"):
        assert ran.get(k, 0) > 0, (k, ran)
    assert "attn_generic" not in ran, ran


# ----------------------------------------------------------------------------- generation through the entry point

@pytest.mark.parametrize("which", ["A", "C"])
def test_greedy_generation_through_the_engine(models, which):
    import mlxforge_b200 as mf
    d, cfg, reqs, expected, _, w = models[(which, False)]
    prompts = [reqs["r1"], reqs["r4"], reqs["r3"][:50]]
    # portions of at most 16 tokens under a budget of 24: prompts are cut and run beside decoding
    eng = mf.Engine(model_spec=d, dtype="float32", kv_pool_tokens=1024, prefill_chunk=16, token_budget=24, max_running=4)
    got = eng.generate(prompts, max_tokens=6)
    clear = agree = 0
    for p, g in zip(prompts, got):
        seq = list(p)
        for t in g:
            row = P.forward(cfg, w, seq)[-1]
            top2 = np.sort(row)[-2:]
            if top2[1] - top2[0] > 1e-3:
                clear += 1
                agree += int(t == int(np.argmax(row)))
            seq.append(t)
    assert clear >= 10 and agree == clear, (got, clear, agree)
    assert eng.metrics()["completed"] == 3
    eng16 = mf.Engine(model_spec=d, dtype="bfloat16", kv_pool_tokens=1024, max_running=4)
    out16 = eng16.generate(prompts, max_tokens=6)
    assert all(len(o) == 6 for o in out16)


def test_cli_generate_and_trace_run_for_luzinex(models, tmp_path, capsys):
    from mlxforge_b200 import cli
    from mlxforge_b200.engine import replay as R
    d, cfg, reqs, expected, tols, w = models[("B", False)]
    prompt_ids = reqs["r2"][:20]
    capsys.readouterr()
    assert cli.main(["generate", d, ",".join(map(str, prompt_ids)), "5", "--dtype", "float32"]) == 0
    got = [int(t) for t in capsys.readouterr().out.split()]
    seq, want = list(prompt_ids), []
    for _ in range(5):
        row = P.forward(cfg, w, seq)[-1]
        want.append(int(np.argmax(row)))
        seq.append(want[-1])
    assert got == want, (got, want)
    trace = TT.mixed(reqs, max_live=4, seed=1, decode_last=4)
    out_dir = tmp_path / "out"
    import sys
    old = sys.stdin
    sys.stdin = trace.lines()
    try:
        assert R.main(["--model", d, "--dtype", "float32", "--out", str(out_dir), "--max-tokens",
                       str(trace.live_tokens_rounded())]) == 0
    finally:
        sys.stdin = old
    capsys.readouterr()
    worst, where = TT.worst(TT.read_outputs(trace, str(out_dir), cfg["vocab"]), expected)
    assert worst <= tols["float32"], (worst, where)


def test_random_weights_mode_writes_a_model_that_loads(tmp_path):
    """The engine's own random-weights mode for this architecture, then a step through the model it wrote."""
    import json
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.engine.replay import make_runner
    from mlxforge_b200.engine.step import StepEntry
    from mlxforge_b200.weights.random_init import write_random_model
    from luzinex_helpers import LZ_A
    d = write_random_model(str(tmp_path / "m"), config_from_json(json.loads(json.dumps(LZ_A))), seed=5, norm_std=0.1)
    runner = make_runner(d, "bfloat16", 64)
    seq = runner.cache.open_sequence()
    logits = runner.step([StepEntry(seq, [1, 2, 3, 4, 5], [4])])
    assert logits.shape == (1, 101) and bool(np.isfinite(host(logits)).all())
