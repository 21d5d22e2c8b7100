"""The Notirax parts and models on the GPU against the plain implementation (plain_notirax.py).

Part by part (each built from its registry with its own sizes, given a runtime, a step batch and a
cache lane, run over portions and single tokens of two sequences), then whole models of three
configurations through the trace replayer's functions -- whole prompts, the last tokens decoded
one by one, portions down to two tokens, mixed batches on a pool so small that pages and slots are
used again, every request decoded from its first token -- in float32 and bfloat16, and greedy
generation through the engine's entry point and scheduler."""
import io
from types import SimpleNamespace

import numpy as np
import pytest

import plain_notirax as P
import trace_tools as TT
from helpers import bf16_round
from notirax_helpers import CONFIGS, make_model, prompt

pytestmark = pytest.mark.gpu

LENGTHS = [45, 23]
STEPS = [(20, 0), (7, 5), (0, 16), (17, 1), (1, 1)]     # tokens of (sequence 0, sequence 1) per step


def tdt(name):
    import torch
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    import torch
    return t.detach().to("cpu", torch.float32).numpy().astype(np.float64)


def tol(dtype, scale):
    return (3e-5 if dtype == "float32" else 3e-2) * max(1.0, scale)


def rand(rng, *shape, std=1.0):
    return bf16_round(rng.standard_normal(shape).astype(np.float32) * std)


class Harness:
    """A runtime, a cache with one lane of the given need and the runner's metadata builder."""

    def __init__(self, dtype, need, lengths=LENGTHS, steps=STEPS, page_size=16, max_tokens=512):
        import torch
        from mlxforge_b200.cache.manager import CacheLayout, CacheManager, GroupLayout
        from mlxforge_b200.engine.runtime import Runtime
        from mlxforge_b200.engine.step import ModelRunner
        from mlxforge_b200.parts.base import PagedKV
        self.rt = Runtime(tdt(dtype))
        paged = isinstance(need, PagedKV)
        layout = CacheLayout(paged=(GroupLayout(need, 1),) if paged else (), state=() if paged else (GroupLayout(need, 1),),
                             item_lane=(("paged" if paged else "state", 0, 0),))
        self.cache = CacheManager(layout, page_size=page_size, max_tokens=max_tokens, max_seqs=4, dtype=tdt(dtype),
                                  device="cuda")
        for pool in self.cache._k + self.cache._v:
            pool.fill_(float("nan"))
        self.cache.open_sequence()                                     # so that the sequences do not sit in slot 0
        for st in self.cache._state:
            st.fill_(float("nan"))                                     # a slot is zeroed when a sequence opens
        stub = SimpleNamespace(graph_safe=False, spec=SimpleNamespace(vocab_size=1 << 20))
        self.runner = ModelRunner(stub, self.cache, self.rt)
        self.lengths, self.plan = lengths, steps
        self.seqs = [self.cache.open_sequence() for _ in lengths]
        torch.cuda.synchronize()

    def steps(self):
        """Yields (batch, rows): rows[i] = (sequence, position) of the step's i-th token."""
        from mlxforge_b200.engine.step import StepEntry
        done = [0] * len(self.lengths)
        for counts in self.plan:
            entries, per_seq = [], []
            for s, n in enumerate(counts):
                if n:
                    entries.append(StepEntry(self.seqs[s], [0] * n, []))
                    per_seq.append((s, n))
            self.cache.reserve([(e.seq, len(e.tokens)) for e in entries])
            batch = self.runner._build(entries)
            order = sorted(range(len(per_seq)), key=lambda i: (per_seq[i][1] != 1, i))
            rows = [(per_seq[i][0], done[per_seq[i][0]] + j) for i in order for j in range(per_seq[i][1])]
            yield batch, rows
            for e in entries:
                self.cache.commit(e.seq, len(e.tokens))
            for s, n in per_seq:
                done[s] += n
        assert done == list(self.lengths)

    def run_mixer(self, part, xs, dtype):
        """The mixer's output for every token of the sequences ``xs`` (arrays [len, H]), fed in steps."""
        got = [np.zeros((len(x), part.hidden)) for x in xs]
        lane = self.cache.lane(0)
        for batch, rows in self.steps():
            x = np.stack([xs[s][p] for s, p in rows])
            out = host(part.forward(dev(x, tdt(dtype)), batch, lane))
            bias = getattr(part, "output_bias", None)
            if bias is not None:
                out = out + host(bias)
            for i, (s, p) in enumerate(rows):
                got[s][p] = out[i]
        return got


# ----------------------------------------------------------------------------- streams, norm, embedding

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,groups,H", [(1, 1, 40), (3, 4, 96), (5, 3, 33 * 3), (8, 2, 2048)])
def test_stream_write_read_and_grouped_norm(dtype, S, groups, H):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(S * 100 + groups)
    T, eps = 7, 1e-5
    x = rng.standard_normal((T, S, H)).astype(np.float32) * 2
    y, bias = rand(rng, T, H), rng.standard_normal(H).astype(np.float32)
    mix = (np.eye(S) + 0.3 * rng.standard_normal((S, S))).astype(np.float32)
    w_out, w_in = rng.standard_normal(S).astype(np.float32), rng.standard_normal(S).astype(np.float32)
    w = (1 + 0.2 * rng.standard_normal(H)).astype(np.float32)
    f = np.float64
    new = P.hyper_write(x.transpose(1, 0, 2).astype(f), y.astype(f) + bias, mix.astype(f), w_out.astype(f))
    want = P.group_rms_norm(P.hyper_read(new, w_in.astype(f)), w.astype(f), eps, groups)
    streams = dev(x.reshape(T, S * H))
    out = torch.empty((T, H), dtype=tdt(dtype), device="cuda")
    ops.hyper_update_norm(streams, dev(y, tdt(dtype)), dev(bias), dev(mix), dev(w_out), dev(w_in), dev(w), eps, groups,
                          out, S)
    assert np.max(np.abs(host(out) - want)) < tol(dtype, np.abs(want).max())
    assert np.max(np.abs(host(streams).reshape(T, S, H).transpose(1, 0, 2) - new)) < 1e-5 * np.abs(new).max()
    # selected rows only: the streams stay, the result is that of the rows; no read weights: the plain sum
    streams = dev(x.reshape(T, S * H))
    rows = dev(np.array([5, 0, 5], dtype=np.int32))
    out = torch.empty((3, H), dtype=tdt(dtype), device="cuda")
    ops.hyper_update_norm(streams, dev(y, tdt(dtype)), None, dev(mix), dev(w_out), None, dev(w), eps, groups, out, S, rows)
    new = P.hyper_write(x.transpose(1, 0, 2).astype(f), y.astype(f), mix.astype(f), w_out.astype(f))
    want = P.group_rms_norm(new.sum(0), w.astype(f), eps, groups)[[5, 0, 5]]
    assert np.max(np.abs(host(out) - want)) < tol(dtype, np.abs(want).max())
    assert np.array_equal(host(streams), x.reshape(T, S * H).astype(f))
    # nothing pending, identity write: the ordinary residual sum
    streams = dev(x.reshape(T, S * H))
    out = torch.empty((T, H), dtype=tdt(dtype), device="cuda")
    ops.hyper_update_norm(streams, None, None, None, None, dev(w_in), dev(w), eps, groups, out, S)
    want = P.group_rms_norm(P.hyper_read(x.transpose(1, 0, 2).astype(f), w_in.astype(f)), w.astype(f), eps, groups)
    assert np.max(np.abs(host(out) - want)) < tol(dtype, np.abs(want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_with_sinusoid_into_every_stream(dtype):
    import torch
    from mlxforge_b200.parts.base import EMBEDDINGS, PartSpec, build_part
    from mlxforge_b200.engine.runtime import Runtime
    rng = np.random.default_rng(0)
    V, H, S = 50, 37, 3
    part = build_part(EMBEDDINGS, PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "tensor": "embed",
                                                               "positions": "sinusoid"}), Runtime(tdt(dtype)))
    table = rand(rng, V, H)
    part.bind({"embed": dev(table)})
    tokens = np.array([3, 49, 0, 7], dtype=np.int32)
    positions = np.array([0, 1, 1500, 40000], dtype=np.int32)
    out = torch.empty((4, S * H), dtype=torch.float32, device="cuda")
    part.embed(SimpleNamespace(tokens=dev(tokens), positions=dev(positions)), out, S)
    want = P.embed(table.astype(np.float64), tokens, positions)
    got = host(out).reshape(4, S, H)
    for s in range(S):
        assert np.max(np.abs(got[:, s] - want)) < (2e-6 if dtype == "float32" else 5e-3)


# ----------------------------------------------------------------------------- attention

ATTN_CASES = {
    # heads, kv, dim, vdim, chunk, window, softcap, talking
    "odd": (6, 2, 24, 40, 7, 0, 4.0, True),
    "page_chunk": (4, 4, 16, 16, 16, 0, 0.0, True),
    "no_talk_no_chunk": (3, 1, 32, 8, 0, 0, 30.0, False),
    "window": (4, 2, 16, 24, 0, 9, 0.0, True),
    "tiles": (4, 2, 64, 64, 40, 0, 10.0, True),
    "long": (4, 2, 64, 32, 0, 0, 10.0, True),        # no chunk and 1,300 tokens: the key range is cut across blocks
    "two_heads": (2, 1, 32, 32, 24, 0, 5.0, True),   # fewer heads than the tensor-core kernel has warps
    "sixteen_heads": (16, 4, 16, 96, 50, 0, 8.0, True),
}
ATTN_PLANS = {"tiles": ([150, 70], [(129, 0), (2, 40), (18, 29), (1, 1)]),
              "long": ([1300, 70], [(1100, 0), (150, 40), (49, 29), (1, 1)])}


def _attention_part(dtype, case, rng, H=56, gain=1.0):
    from mlxforge_b200.parts.base import MIXERS, PartSpec, build_part
    nh, nkv, d, dv, chunk, window, cap, talking = ATTN_CASES[case]
    params = {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d, "v_head_dim": dv,
              "softmax_scale": 1.7 * d ** -0.5, "softcap": cap, "talking": talking, "chunk": chunk, "window": window}
    part = build_part(MIXERS, PartSpec("talking_attention", params, prefix="a."), None)
    w = {}
    for name, spec in part.tensor_specs().items():
        if name.endswith("talk"):
            w[name] = bf16_round((np.eye(nh) + 0.3 * rng.standard_normal((nh, nh))).astype(np.float32))
        elif len(spec.shape) == 1:
            w[name] = rand(rng, *spec.shape, std=0.3)
        else:
            g = gain if name in ("a.q", "a.k") else 1.0
            w[name] = rand(rng, *spec.shape, std=g / np.sqrt(spec.shape[1]))
    p = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": dv, "scale": params["softmax_scale"], "softcap": cap,
         "mask": {"size": chunk} if chunk else None}
    return params, w, p, window


def _plain_attention(x, p, w, window):
    f = {k[2:]: v.astype(np.float64) for k, v in w.items()}
    if not window:
        return P.talking_chunk_attention(x, p, f.get)
    # a window is not in the plain model: the same function on every window's keys alone
    out = np.zeros((x.shape[0], f["o"].shape[0]))
    q_only = dict(p)
    for i in range(x.shape[0]):
        lo = max(0, i - window + 1)
        out[i] = P.talking_chunk_attention(x[lo:i + 1], q_only, f.get)[-1]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(ATTN_CASES))
def test_talking_attention_part(dtype, case):
    from mlxforge_b200.parts.base import MIXERS, PartSpec, build_part
    rng = np.random.default_rng(sum(map(ord, case)))
    params, w, p, window = _attention_part(dtype, case, rng)
    lengths, steps = ATTN_PLANS.get(case, (LENGTHS, STEPS))
    part = build_part(MIXERS, PartSpec("talking_attention", params, prefix="a."), None)
    need = part.cache_need()
    h = Harness(dtype, need, lengths, steps, max_tokens=2048)
    part = build_part(MIXERS, PartSpec("talking_attention", params, prefix="a."), h.rt)
    part.bind({n: dev(a) for n, a in w.items()})
    xs = [rand(rng, n, params["hidden_size"]) for n in lengths]
    got = h.run_mixer(part, xs, dtype)
    for s, x in enumerate(xs):
        want = _plain_attention(x.astype(np.float64), p, w, window)
        assert np.max(np.abs(got[s] - want)) < tol(dtype, np.abs(want).max()), (case, s)
    if params["chunk"]:
        # pages before the chunk of the next query went back to the pool
        held = h.seqs[0].pages_held(0)
        assert held == (lengths[0] + 15) // 16 - (lengths[0] // params["chunk"] * params["chunk"]) // 16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["odd", "page_chunk", "tiles"])
def test_keys_at_the_edges_of_chunks_and_pages_decide(dtype, case):
    """The keys at the last place of a chunk, the first of the next, and at both sides of every page
    border are made to stand out (their scores are far above the others'), with values of their own:
    a query that sees one key too many or too few ends somewhere else.  In prompts and decoding."""
    from mlxforge_b200.parts.base import MIXERS, PartSpec, build_part
    rng = np.random.default_rng(5)
    params, w, p, window = _attention_part(dtype, case, rng, gain=1.0)
    chunk, H = params["chunk"], params["hidden_size"]
    lengths = [4 * chunk + 3, 2 * chunk + 1] if chunk < 30 else [150, 90]
    steps = [(lengths[0] - chunk - 2, 3), (2, lengths[1] - 5)] + [(1, 1)] * 2 + [(chunk - 2, 0)]
    steps[-1] = (lengths[0] - sum(s[0] for s in steps[:-1]), lengths[1] - sum(s[1] for s in steps[:-1]))
    part = build_part(MIXERS, PartSpec("talking_attention", params, prefix="a."), None)
    h = Harness(dtype, part.cache_need(), lengths, steps)
    part = build_part(MIXERS, PartSpec("talking_attention", params, prefix="a."), h.rt)
    # every token's input has a common direction e: queries and keys both project it strongly for the
    # edge tokens, so an edge key outweighs all others for every later query of its chunk
    e = rand(rng, H)
    xs = []
    for n in lengths:
        x = rand(rng, n, H, std=0.3)
        for j in range(n):
            if chunk and (j % chunk in (0, chunk - 1)) or j % 16 in (0, 15):
                x[j] = bf16_round(x[j] + 1.5 * e)
        xs.append(x)
    part.bind({n: dev(a) for n, a in w.items()})
    got = h.run_mixer(part, xs, dtype)
    for s, x in enumerate(xs):
        want = _plain_attention(x.astype(np.float64), p, w, window)
        assert np.max(np.abs(got[s] - want)) < tol(dtype, np.abs(want).max()), (case, s)


# ----------------------------------------------------------------------------- gated delta rule

DELTA_CASES = {
    # heads, kv, dim, vdim, taps, decay rank, gate rank
    "odd": (6, 2, 20, 12, 4, 5, 3),
    "one_tap": (2, 2, 16, 16, 1, 4, 4),
    "wide": (2, 1, 128, 48, 2, 8, 8),
    "long_taps": (3, 3, 40, 24, 6, 2, 7),
    "unaligned": (2, 1, 18, 10, 3, 3, 3),            # sizes that are no multiple of 4: the kernel without 16-byte copies
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(DELTA_CASES))
def test_channel_delta_part(dtype, case):
    from mlxforge_b200.parts.base import MIXERS, PartSpec, build_part
    rng = np.random.default_rng(len(case))
    nh, nkv, d, dv, taps, ra, rg = DELTA_CASES[case]
    H, eps = 48, 1e-5
    params = {"hidden_size": H, "n_heads": nh, "n_kv_heads": nkv, "head_dim": d, "v_head_dim": dv, "conv": taps,
              "eps": eps, "decay_rank": ra, "gate_rank": rg}
    part = build_part(MIXERS, PartSpec("channel_delta", params, prefix="m."), None)
    # portions shorter than the convolution's history, single tokens in between
    lengths, steps = [60, 31], [(20, 0), (2, 5), (1, 1), (1, 0), (3, 16), (17, 1), (1, 1), (15, 7)]
    h = Harness(dtype, part.cache_need(), lengths, steps)
    part = build_part(MIXERS, PartSpec("channel_delta", params, prefix="m."), h.rt)
    w = {}
    for name, spec in part.tensor_specs().items():
        leaf = name.split(".")[-1]
        if leaf == "norm":
            w[name] = bf16_round((1 + 0.1 * rng.standard_normal(spec.shape)).astype(np.float32))
        elif leaf in ("conv", "A_log", "dt_bias"):
            w[name] = rand(rng, *spec.shape, std=0.6)
        else:
            w[name] = rand(rng, *spec.shape, std=1.5 / np.sqrt(spec.shape[1]))
    part.bind({n: dev(a) for n, a in w.items()})
    xs = [rand(rng, n, H) for n in lengths]
    got = h.run_mixer(part, xs, dtype)
    p = {"heads": nh, "kv_heads": nkv, "dim": d, "vdim": dv, "conv": taps}
    f = {k[2:]: v.astype(np.float64) for k, v in w.items()}
    for s, x in enumerate(xs):
        want = P.channel_delta(x.astype(np.float64), p, f.get, eps)
        assert np.max(np.abs(got[s] - want)) < tol(dtype, np.abs(want).max()), (case, s)


def test_delta_state_carries_a_far_token():
    """One early token writes into key channels that no other token touches (their keys are zero
    there), the state hardly decays, and the last token asks with a query in those channels: its
    read-out is the early token's value, hundreds of tokens and several steps later.  A state that
    is lost, restarted or decayed wrongly shows."""
    from mlxforge_b200.parts.base import MIXERS, PartSpec, build_part
    rng = np.random.default_rng(9)
    nh, d, dv, H = 2, 16, 16, 32
    params = {"hidden_size": H, "n_heads": nh, "n_kv_heads": nh, "head_dim": d, "v_head_dim": dv, "conv": 1,
              "eps": 1e-6, "decay_rank": 2, "gate_rank": 2}
    part = build_part(MIXERS, PartSpec("channel_delta", params, prefix="m."), None)
    lengths = [300, 5]
    steps = [(100, 1), (1, 1), (50, 1), (2, 1), (146, 1), (1, 0)]
    h = Harness("float32", part.cache_need(), lengths, steps)
    part = build_part(MIXERS, PartSpec("channel_delta", params, prefix="m."), h.rt)
    w = {n: rand(rng, *s.shape, std=0.3 if len(s.shape) > 1 else 0.1) for n, s in part.tensor_specs().items()}
    w["m.a1"] *= 0.0
    w["m.dt_bias"] = np.full(nh * d, -14.0, dtype=np.float32)            # softplus ~ 1e-6: the state hardly decays
    w["m.q.conv"], w["m.k.conv"], w["m.v.conv"] = (np.ones_like(w[n]) for n in ("m.q.conv", "m.k.conv", "m.v.conv"))
    w["m.norm"] = np.ones(dv, dtype=np.float32)
    # ordinary tokens live in the first half of the width; the second half is read by the upper key
    # and query channels of every head only, and by nothing else of q and k
    for n in ("m.q", "m.k"):
        m = w[n].reshape(nh, d, H)
        m[:, :d // 2, H // 2:] = 0.0
        m[:, d // 2:, :H // 2] = 0.0
        m[:, d // 2:, H // 2:] = np.abs(m[:, d // 2:, H // 2:])
    xs = [rand(rng, n, H, std=0.5) for n in lengths]
    for x in xs:
        x[:, H // 2:] = 0.0
    e = np.zeros(H, dtype=np.float32)
    e[H // 2:] = bf16_round(np.abs(rng.standard_normal(H // 2)).astype(np.float32) + 1.0)
    xs[0][3] += e                                                        # the far token
    xs[0][299] += e                                                      # the query that asks for it
    part.bind({n: dev(a) for n, a in w.items()})
    got = h.run_mixer(part, xs, "float32")
    p = {"heads": nh, "kv_heads": nh, "dim": d, "vdim": dv, "conv": 1}
    f = {k[2:]: v.astype(np.float64) for k, v in w.items()}
    want = P.channel_delta(xs[0].astype(np.float64), p, f.get, 1e-6)
    without = xs[0].astype(np.float64).copy()
    without[3] -= e
    assert np.max(np.abs(P.channel_delta(without, p, f.get, 1e-6)[299] - want[299])) > 0.2 * np.abs(want[299]).max(), \
        "the far token does not decide: the test would show nothing"
    assert np.max(np.abs(got[0] - want)) < 3e-5 * max(1.0, np.abs(want).max())


# ----------------------------------------------------------------------------- mixture of experts

@pytest.mark.parametrize("E,groups,keep,top", [(12, 4, 2, 3), (8, 0, 0, 2), (6, 6, 3, 2), (64, 8, 3, 6), (4, 1, 1, 4),
                                               (160, 8, 3, 8)])
def test_router_kernel(E, groups, keep, top):
    import torch
    from mlxforge_b200.csrc import ops
    rng = np.random.default_rng(E)
    T = 301
    z = (rng.standard_normal((T, E)) * 2).astype(np.float32)
    ids = torch.empty((T, top), dtype=torch.int32, device="cuda")
    wts = torch.empty((T, top), dtype=torch.float32, device="cuda")
    ops.moe_route(dev(z), groups, keep, top, 1.5, ids, wts)
    r = {"top": top, "scale": 1.5}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    chosen, weight = P.grouped_router(z.astype(np.float64), np.eye(E), r)
    assert np.array_equal(ids.cpu().numpy(), chosen)
    assert np.max(np.abs(wts.cpu().numpy() - weight)) < 1e-6
    if groups > 1 and keep < groups and E // groups > 1:      # with one expert a group the rule cannot change a choice
        free, _ = P.grouped_router(z.astype(np.float64), np.eye(E), {"top": top, "scale": 1.5})
        assert (np.sort(free, -1) != np.sort(chosen, -1)).any(-1).mean() > 0.1, "the groups never decide in this test"


@pytest.mark.parametrize("own_tiles", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,ff,E,groups,keep,top,T", [(40, 24, 6, 3, 2, 2, 9), (64, 64, 8, 0, 0, 3, 150),
                                                       (128, 32, 16, 4, 2, 4, 300), (72, 20, 5, 0, 0, 1, 70)])
def test_routed_experts_part(dtype, H, ff, E, groups, keep, top, T, own_tiles, monkeypatch):
    """``own_tiles``: many tokens in bfloat16 through this engine's own tensor-core tiles instead of the
    library's grouped product (the other cases take the same kernels either way)."""
    from mlxforge_b200.csrc import binding
    from mlxforge_b200.engine.runtime import Runtime
    if own_tiles and (dtype != "bfloat16" or T < 64 or H % 8 or ff % 8):
        pytest.skip("the path does not differ here")
    monkeypatch.setenv("MLXFORGE_MOE_TILES", "1" if own_tiles else "0")
    before = binding.kernel_launches()
    from mlxforge_b200.parts.base import FEED_FORWARDS, PartSpec, build_part
    rng = np.random.default_rng(H + T)
    params = {"hidden_size": H, "intermediate_size": ff, "n_experts": E, "top": top, "n_groups": groups,
              "keep_groups": keep, "route_scale": 1.3, "limit": 0.8}
    part = build_part(FEED_FORWARDS, PartSpec("routed_experts", params, prefix="f."), Runtime(tdt(dtype)))
    w = {n: rand(rng, *s.shape, std=(4.0 if n.endswith("router") else 1.5) / np.sqrt(s.shape[1]))
         for n, s in part.tensor_specs().items()}
    part.bind({n: dev(a) for n, a in w.items()})
    x = rand(rng, T, H)
    p = {"expert": {"limit": 0.8}, "router": {"top": top, "scale": 1.3}}
    if groups:
        p["router"]["groups"] = {"count": groups, "keep": keep}
    f = {k[2:]: v.astype(np.float64) for k, v in w.items()}
    want = P.moe(x.astype(np.float64), p, f.get)
    got = host(part.forward(dev(x, tdt(dtype)), None))
    # a token whose choice hangs on a close call may differ in bfloat16 (the router reads the same
    # bfloat16 inputs, so here it does not); all others must agree
    assert np.max(np.abs(got - want)) < tol(dtype, np.abs(want).max())
    ran = {k: v - before[k] for k, v in binding.kernel_launches().items() if v - before[k]}
    if dtype == "bfloat16" and T >= 64 and H % 8 == 0 and ff % 8 == 0:
        assert ran.get("moe_grouped", 0) == (2 if own_tiles else 2) and ran.get("moe_sort", 0) == 1, ran
    else:
        assert ran.get("moe_rows", 0) == 1, ran
    # each token alone gives the same as inside the batch
    alone = host(part.forward(dev(x[7:8], tdt(dtype)), None))
    assert np.max(np.abs(alone[0] - got[7])) < (1e-5 if dtype == "float32" else 2e-2) * max(1.0, np.abs(want).max())


# ----------------------------------------------------------------------------- whole models through the replayer

REQUEST_LENGTHS = {"A": [1, 9, 40, 75, 131, 58], "B": [2, 17, 33, 64, 100], "C": [300, 45, 520, 203]}
PORTIONS = {"A": (7, 2, 5, 3, 2, 11, 4, 2, 16, 1, 9), "B": (7, 2, 5, 3, 2, 11, 4, 2, 16, 1, 9),
            "C": (150, 2, 129, 7, 64, 3, 131, 200)}
PEAKED = {"A": 6.0, "B": 6.0, "C": 3.0}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("notirax")
    out = {}
    for which in CONFIGS:
        for peaked in (False, True):
            d, cfg, w = make_model(tmp, which, seed=ord(which), qk_gain=PEAKED[which] if peaked else 1.0)
            reqs = {f"r{i}": prompt(cfg, n, i) for i, n in enumerate(REQUEST_LENGTHS[which])}
            expected = {rid: P.forward(cfg, w, toks) for rid, toks in reqs.items()}
            P.ROUND = P.round_bf16
            try:
                noise = max(float(np.max(np.abs(P.forward(cfg, w, toks) - expected[rid]))) for rid, toks in reqs.items())
            finally:
                P.ROUND = None
            scale = max(float(np.max(np.abs(e))) for e in expected.values())
            out[(which, peaked)] = (d, cfg, reqs, expected, {"float32": 1e-4 * max(1.0, scale), "bfloat16": 3.0 * noise}, w)
    return out


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
    worst, where = TT.worst(got, expected)
    assert worst <= tols[dtype], (which, peaked, dtype, worst, tols[dtype], where, TT.first_bad(got, expected, tols[dtype]))
    return ran


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("peaked", [False, True])
@pytest.mark.parametrize("which", list(CONFIGS))
def test_whole_prompts_and_decoded_tails(models, which, peaked, dtype, tmp_path):
    reqs = models[(which, peaked)][2]
    _check(models, which, peaked, dtype, TT.whole(reqs), tmp_path)
    _check(models, which, peaked, dtype, TT.decode_tail(reqs, tail=32), tmp_path / "tail")


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
def test_every_request_decoded_from_its_first_token(models, which, dtype, tmp_path):
    """Long decoding in a batch that shrinks: the first tokens of a sequence, chunk edges and page
    borders met token by token, decode steps replayed from graphs."""
    reqs = models[(which, False)][2]
    _check(models, which, False, dtype, TT.lockstep(reqs), tmp_path, max_seqs=len(reqs))


@pytest.mark.parametrize("own_tiles", [False, True])
def test_serving_shapes_take_the_fast_kernels(models, tmp_path, own_tiles, monkeypatch):
    """Configuration C in bfloat16: which kernels its prompts and its decoding go through, with the experts of
    many tokens through the library's grouped product and through this engine's own tiles."""
    monkeypatch.setenv("MLXFORGE_MOE_TILES", "1" if own_tiles else "0")
    reqs = models[("C", False)][2]
    ran = _check(models, "C", False, "bfloat16", TT.decode_tail(reqs, tail=8), tmp_path)
    for k in ("hyper_norm", "delta_recurrence", "moe_route", "embed_positions", "kv_store"):
        assert ran.get(k, 0) > 0, (k, ran)
    assert ran.get("attn_talking_tc", 0) > 0 and ran.get("attn_talking_merge", 0) > 0, ran
    assert ran.get("moe_grouped", 0) > 0 and ran.get("moe_rows", 0) > 0, ran


# ----------------------------------------------------------------------------- generation through the entry point

@pytest.mark.parametrize("which", ["A", "C"])
def test_greedy_generation_through_the_engine(models, which):
    import mlxforge_b200 as mf
    d, cfg, reqs, expected, _, w = models[(which, False)]
    prompts = [reqs["r2"], reqs["r1"], reqs["r3"][:50]]
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


def test_cli_generate_and_trace_run_for_notirax(models, tmp_path, capsys):
    """The command line's own entry points: `generate` prints the plain implementation's greedy tokens, and the
    replayer's program (four slots unless told otherwise) writes the logits of a small trace."""
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
