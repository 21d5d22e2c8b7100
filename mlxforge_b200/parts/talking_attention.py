"""Attention whose heads talk to each other before the softmax, with a chunk-local mask.

``q = Wq x + bq``, ``k = Wk x + bk``, ``v = Wv x + bv`` (``n_heads`` query heads and ``n_kv_heads``
key/value heads; keys ``head_dim`` wide, values ``v_head_dim``), no position encoding, then

    s_h  = (q_h . k_g(h)) * softmax_scale              g(h) = h // (n_heads / n_kv_heads)
    s_h <- softcap * tanh(s_h / softcap)               (softcap > 0)
    s_h <- sum_g talk[h, g] s_g                        (talking = True: a matrix [n_heads, n_heads])
    p_h  = softmax of s_h over the keys the query sees
    out  = Wo concat_h(p_h v_g(h)) + bo

A query at position ``i`` sees ``j <= i``, limited to its own chunk (``chunk`` > 0:
``floor(j / chunk) == floor(i / chunk)``, chunks counted from position 0 of the sequence) and/or to
a sliding ``window``.  The cache gives back the pages that no later query can see.  Scores, the
mixing and the softmax are 32-bit; the projections' biases are added in 32-bit before the one
rounding to the compute dtype; the output projection's bias is handed to the stream write
(``output_bias``).  Every constant is a parameter; ``names`` maps the roles of the tensors to
their names behind the prefix.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Mixer, PagedKV, TensorSpec, register_mixer

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "talk": "talk", "bias": ".b"}


@register_mixer("talking_attention")
class TalkingAttention(Mixer):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.scale = float(p["softmax_scale"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.talking = bool(p.get("talking", True))
        self.chunk = int(p.get("chunk") or 0)
        self.window = int(p.get("window") or 0)
        self.bias = bool(p.get("bias", True))
        self.names = dict(_NAMES, **(p.get("names") or {}))
        if self.n_kv <= 0 or self.n_heads % self.n_kv:
            raise ValueError("talking_attention: n_heads must be a multiple of n_kv_heads")
        if self.chunk < 0 or self.window < 0 or self.softcap < 0:
            raise ValueError("talking_attention: chunk, window and softcap must not be negative")
        self.w_qkv = self.b_qkv = self.w_o = self.output_bias = self.talk = None

    def _n(self, role: str, bias: bool = False) -> str:
        return self.prefix + self.names[role] + (self.names["bias"] if bias else "")

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nq, nk, nv = self.n_heads * self.dim, self.n_kv * self.dim, self.n_kv * self.vdim
        specs = {self._n("q"): TensorSpec((nq, self.hidden)), self._n("k"): TensorSpec((nk, self.hidden)),
                 self._n("v"): TensorSpec((nv, self.hidden)), self._n("o"): TensorSpec((self.hidden, self.n_heads * self.vdim))}
        if self.bias:
            for role, n in (("q", nq), ("k", nk), ("v", nv), ("o", self.hidden)):
                specs[self._n(role, True)] = TensorSpec((n,), role="vector")
        if self.talking:
            specs[self._n("talk")] = TensorSpec((self.n_heads, self.n_heads), role="vector")
        return specs

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        self.w_qkv = torch.cat([tensors[self._n(r)].to(dt) for r in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        if self.bias:
            self.b_qkv = torch.cat([tensors[self._n(r, True)].to(torch.float32) for r in ("q", "k", "v")]).contiguous()
            self.output_bias = tensors[self._n("o", True)].to(torch.float32).contiguous()
        if self.talking:
            self.talk = tensors[self._n("talk")].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()

    def cache_need(self):
        return PagedKV(self.n_kv, self.dim, self.window, self.chunk, self.vdim if self.vdim != self.dim else 0)

    def project(self, x):
        """[T, H] -> queries, keys and values side by side in 32-bit (the biases are still to come)."""
        T = x.shape[0]
        n = self.n_heads * self.dim + self.n_kv * (self.dim + self.vdim)
        return self.rt.linear(x, self.w_qkv, self.rt.buffer("tattn.qkv", (T, n), torch.float32))

    def encode_and_store(self, qkv, batch, cache, writes_cache: bool):
        q = self.rt.buffer("tattn.q", (qkv.shape[0], self.n_heads * self.dim))
        cache.store(qkv, batch, q, self.n_heads, self.n_kv, writes_cache, precise=self.rt.precise, bias=self.b_qkv)
        return q

    def attend(self, q, batch, cache):
        o = self.rt.buffer("tattn.o", (q.shape[0], self.n_heads * self.vdim))
        talking_paged_attention(self.rt, batch, q, cache, o, self)
        return o

    def output(self, o):
        return self.rt.linear(o, self.w_o, self.rt.buffer("tattn.delta", (o.shape[0], self.hidden)))

    def forward(self, x, batch, cache, writes_cache: bool = True):
        qkv = self.project(x)
        q = self.encode_and_store(qkv, batch, cache, writes_cache)
        return self.output(self.attend(q, batch, cache))


def talking_paged_attention(rt, batch, q, lane, out, m: TalkingAttention) -> None:
    """The kernel is chosen by dtype and by how many tokens a sequence brings, as for the plain
    attention.  bfloat16 with sizes the tensor-core kernel takes: the sequences that bring one token
    (the batch lays them out first) go through it with their keys cut into splits and a merge, the
    portions of prompts with a block per 16 queries.  Everything else (the 32-bit path, other
    sizes) takes the kernel with a block per token."""
    table = batch.block_table(lane.group)
    tc = q.dtype == torch.bfloat16 and ops.attention_talking_tc_ok(m.n_heads, m.n_kv, m.dim, m.vdim, lane.page_size)
    if not tc:
        ops.attention_talking(q, lane.k, lane.v, out, batch.positions, batch.seq_of_token, table, lane.page_size,
                              m.n_heads, m.n_kv, m.dim, m.vdim, m.scale, m.softcap, m.talk, m.window, m.chunk)
        return
    nd = batch.n_decode
    max_keys = batch.max_ctx
    if m.chunk:
        max_keys = min(max_keys, m.chunk)
    if m.window:
        max_keys = min(max_keys, m.window)
    if nd > 0:
        splits = ops.attention_talking_splits(max_keys)
        part_o = rt.buffer("tattn.part_o", (nd * splits * m.n_heads * m.vdim,), torch.float32)
        part_ml = rt.buffer("tattn.part_ml", (nd * splits * m.n_heads * 2,), torch.float32)
        ops.attention_talking_decode(q[:nd], lane.k, lane.v, out[:nd], batch.seq_q_start[:nd], batch.seq_q_len[:nd],
                                     batch.seq_ctx_len[:nd], table, lane.page_size, m.n_heads, m.n_kv, m.dim, m.vdim,
                                     m.scale, m.softcap, m.talk, m.window, m.chunk, splits, part_o, part_ml)
    if nd < batch.n_tokens:
        T = batch.n_tokens
        splits = ops.attention_talking_prefill_splits(max_keys)
        part_o = part_ml = None
        if splits:
            part_o = rt.buffer("tattn.part_o", (T * splits * m.n_heads * m.vdim,), torch.float32)
            part_ml = rt.buffer("tattn.part_ml", (T * splits * m.n_heads * 2,), torch.float32)
        ops.attention_talking_tc(q, lane.k, lane.v, out, batch.seq_q_start[nd:], batch.seq_q_len[nd:],
                                 batch.seq_ctx_len[nd:], nd, max(batch.q_len[nd:]), table, lane.page_size,
                                 m.n_heads, m.n_kv, m.dim, m.vdim, m.scale, m.softcap, m.talk, m.window, m.chunk,
                                 splits, part_o, part_ml, nd)
