"""Gated delta rule with a decay per head and key channel ("channel delta"), a recurrent mixer.

Per head, with a 32-bit state ``S`` [head_dim, v_head_dim] per request, token after token:

    S <- diag(g_t) S ;   u = beta_t (v_t - S^T k_t) ;   S <- S + k_t u^T ;   o_t = S^T q_t

``q, k`` (``n_kv_heads`` heads) and ``v`` (``n_heads`` heads) are projections of the input, each
through a short causal convolution over time per channel (``conv`` taps, the last one the current
token's, zeros before the start) and SiLU; ``q`` and ``k`` are made unit vectors per head
(``x / sqrt(sum x^2 + 1e-6)``), ``q`` also times ``head_dim^-1/2``; head ``h`` uses q/k head
``h // (n_heads / n_kv_heads)``.  ``beta = sigmoid(Wb x)`` per head;
``g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 x) + dt_bias))`` per head and key channel.  The read-out of
every head is divided by its root mean square over ``v_head_dim`` (``eps``), multiplied by a weight
shared by the heads and by ``sigmoid(Wg2 (Wg1 x))``, then projected by ``Wo``.

The request's slot keeps ``S`` of every head and the last ``conv - 1`` inputs of every convolution,
so a step goes on from where the step before ended, however the prompt was cut.  All projections
that read the mixer's input are one product; the two low-rank second factors are one product with a
block-diagonal matrix.  Everything after the projections is 32-bit.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FixedState, Mixer, TensorSpec, register_mixer

_NAMES = {"q": "q", "k": "k", "v": "v", "conv": ".conv", "beta": "b", "A_log": "A_log", "dt_bias": "dt_bias",
          "a1": "a1", "a2": "a2", "g1": "g1", "g2": "g2", "norm": "norm", "o": "o"}


@register_mixer("channel_delta")
class ChannelDeltaMixer(Mixer):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p.get("v_head_dim") or self.dim)
        self.taps = int(p["conv"])
        self.eps = float(p["eps"])
        self.decay_rank = int(p["decay_rank"])
        self.gate_rank = int(p["gate_rank"])
        self.names = dict(_NAMES, **(p.get("names") or {}))
        if self.n_kv <= 0 or self.n_heads % self.n_kv:
            raise ValueError("channel_delta: n_heads must be a multiple of n_kv_heads")
        if self.taps < 1:
            raise ValueError("channel_delta: conv must be at least 1 tap")
        if self.dim > 256:
            raise ValueError(f"channel_delta: head_dim {self.dim} is larger than the recurrence kernel's 256")
        self.channels = 2 * self.n_kv * self.dim + self.n_heads * self.vdim
        self.state_floats = self.n_heads * self.dim * self.vdim
        self.w_in = self.w_low = self.w_o = self.conv_w = self.a_log = self.dt_bias = self.norm_w = None

    def _n(self, role: str) -> str:
        return self.prefix + self.names[role]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nqk, nv, H = self.n_kv * self.dim, self.n_heads * self.vdim, self.hidden
        c = self.names["conv"]
        return {
            self._n("q"): TensorSpec((nqk, H)), self._n("k"): TensorSpec((nqk, H)), self._n("v"): TensorSpec((nv, H)),
            self._n("q") + c: TensorSpec((nqk, self.taps), role="vector"),
            self._n("k") + c: TensorSpec((nqk, self.taps), role="vector"),
            self._n("v") + c: TensorSpec((nv, self.taps), role="vector"),
            self._n("beta"): TensorSpec((self.n_heads, H)),
            self._n("A_log"): TensorSpec((self.n_heads,), role="vector"),
            self._n("dt_bias"): TensorSpec((self.n_heads * self.dim,), role="vector"),
            self._n("a1"): TensorSpec((self.decay_rank, H)), self._n("a2"): TensorSpec((self.n_heads * self.dim, self.decay_rank)),
            self._n("g1"): TensorSpec((self.gate_rank, H)), self._n("g2"): TensorSpec((nv, self.gate_rank)),
            self._n("norm"): TensorSpec((self.vdim,), role="vector"),
            self._n("o"): TensorSpec((H, nv)),
        }

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        f32 = torch.float32
        c = self.names["conv"]
        self.w_in = torch.cat([tensors[self._n(r)].to(dt) for r in ("q", "k", "v", "beta", "a1", "g1")], dim=0).contiguous()
        a2, g2 = tensors[self._n("a2")].to(dt), tensors[self._n("g2")].to(dt)
        low = torch.zeros((a2.shape[0] + g2.shape[0], self.decay_rank + self.gate_rank), dtype=dt, device=a2.device)
        low[:a2.shape[0], :self.decay_rank] = a2
        low[a2.shape[0]:, self.decay_rank:] = g2
        self.w_low = low.contiguous()
        self.w_o = tensors[self._n("o")].to(dt).contiguous()
        self.conv_w = torch.cat([tensors[self._n(r) + c].to(f32) for r in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = tensors[self._n("A_log")].to(f32).contiguous()
        self.dt_bias = tensors[self._n("dt_bias")].to(f32).contiguous()
        self.norm_w = tensors[self._n("norm")].to(f32).contiguous()

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_low.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_need(self):
        return FixedState((self.state_floats + (self.taps - 1) * self.channels,), tag="channel_delta")

    def forward(self, x, batch, cache, writes_cache: bool = True):
        rt, T = self.rt, x.shape[0]
        f32 = torch.float32
        nh, nkv, d, dv = self.n_heads, self.n_kv, self.dim, self.vdim
        state = cache.tensor                                       # [slots, S of every head | convolution tails]
        proj = rt.linear(x, self.w_in, rt.buffer("delta.proj", (T, self.w_in.shape[0]), f32))
        qkv = rt.buffer("delta.qkv", (T, self.channels), f32)
        beta = rt.buffer("delta.beta", (T, nh), f32)
        low = rt.buffer("delta.low", (T, self.decay_rank + self.gate_rank))
        ops.delta_prepare(proj, self.conv_w, self.taps, state, self.state_floats, batch, qkv, beta, low, nh, nkv, d, dv)
        ag = rt.linear(low, self.w_low, rt.buffer("delta.ag", (T, nh * d + nh * dv), f32))
        ops.delta_gates(ag, self.a_log, self.dt_bias, nh, d, nh * dv)
        o = rt.buffer("delta.o", (T, nh * dv), f32)
        ops.delta_recurrence(qkv, beta, ag, state, batch, o, nh, nkv, d, dv)
        og = rt.buffer("delta.og", (T, nh * dv))
        ops.delta_output(o, ag[:, nh * d:], ag.shape[1], self.norm_w, self.eps, og, nh, dv)
        return rt.linear(og, self.w_o, rt.buffer("delta.delta", (T, self.hidden)))
