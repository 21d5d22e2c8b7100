"""Mixture of experts with a sigmoid router that is limited to the best groups of experts.

Router (32-bit): ``s = sigmoid(Wr x)``.  The ``n_experts`` experts form ``n_groups`` equal groups
of neighbours; a group's score is the sum of its two largest ``s``, and only experts of the
``keep_groups`` best groups can be chosen (``n_groups`` = 0: any expert).  Each token uses the
``top`` allowed experts with the largest ``s``, weighted by ``s * route_scale`` (not renormalised);
ties go to the lower index.  Expert ``e``:

    g = min(Wg_e x, limit) ;  u = clamp(Wu_e x, -limit, limit) ;  y = Wd_e (g sigmoid(alpha g) (u + 1))

The experts' matrices are stacked at load time (``[E, 2, ff, H]`` gate rows then up rows, and
``[E, H, ff]``).  Few tokens (and the 32-bit path) take the kernel with a block per (token, chosen
expert), which streams that expert's matrices once; many tokens in bfloat16 are sorted by expert
and go through the library's grouped product (as the engine's other many-row products go through
the library) with this engine's gather, activation and weighted-sum kernels around it, or, where
nothing may be allocated (a CUDA graph being recorded), the library lacks it, or the backend is
``tcgen05``/``MLXFORGE_MOE_TILES=1``, through this engine's own tensor-core tiles.  Either way a
token's chosen experts are added in the order of the choice, so its result does not depend on what
else is in the batch.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, TensorSpec, register_feed_forward

_NAMES = {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden = int(p["hidden_size"])
        self.ff = int(p["intermediate_size"])
        self.n_experts = int(p["n_experts"])
        self.top = int(p["top"])
        self.n_groups = int(p.get("n_groups") or 0)
        self.keep = int(p.get("keep_groups") or 0)
        self.route_scale = float(p.get("route_scale", 1.0))
        self.limit = float(p["limit"])
        self.alpha = float(p.get("alpha", 1.702))
        self.names = dict(_NAMES, **(p.get("names") or {}))
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"routed_experts: top {self.top} of {self.n_experts} experts")
        if self.n_groups:
            if self.n_experts % self.n_groups or not (1 <= self.keep <= self.n_groups):
                raise ValueError(f"routed_experts: {self.n_experts} experts, {self.n_groups} groups, keep {self.keep}")
            if self.keep * (self.n_experts // self.n_groups) < self.top:
                raise ValueError("routed_experts: the kept groups hold fewer experts than a token uses")
        # tokens from which the sorted, tiled path is taken (bfloat16 only)
        self.grouped_min_tokens = int(p.get("grouped_min_tokens", 64))
        self.w_router = self.w_gu = self.w_down = None

    def _e(self, e: int, role: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[role]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = {self.prefix + self.names["router"]: TensorSpec((self.n_experts, self.hidden))}
        for e in range(self.n_experts):
            specs[self._e(e, "gate")] = TensorSpec((self.ff, self.hidden))
            specs[self._e(e, "up")] = TensorSpec((self.ff, self.hidden))
            specs[self._e(e, "down")] = TensorSpec((self.hidden, self.ff))
        return specs

    def bind(self, tensors) -> None:
        dt = self.rt.dtype
        self.w_router = tensors[self.prefix + self.names["router"]].to(dt).contiguous()
        self.w_gu = torch.stack([torch.stack([tensors[self._e(e, "gate")].to(dt), tensors[self._e(e, "up")].to(dt)])
                                 for e in range(self.n_experts)]).contiguous()           # [E, 2, ff, H]
        self.w_down = torch.stack([tensors[self._e(e, "down")].to(dt) for e in range(self.n_experts)]).contiguous()

    def weight_bytes(self) -> int:
        # a step reads the router and, per token, `top` experts; at most all of them
        per = 3 * self.ff * self.hidden * self.w_gu.element_size()
        return self.w_router.numel() * self.w_router.element_size() + self.n_experts * per

    def route(self, x):
        T = x.shape[0]
        z = self.rt.linear(x, self.w_router, self.rt.buffer("moe.z", (T, self.n_experts), torch.float32))
        ids = self.rt.buffer("moe.ids", (T, self.top), torch.int32)
        weights = self.rt.buffer("moe.weights", (T, self.top), torch.float32)
        ops.moe_route(z, self.n_groups, self.keep, self.top, self.route_scale, ids, weights)
        return ids, weights

    def forward(self, x, batch):
        rt, T = self.rt, x.shape[0]
        ids, weights = self.route(x)
        out = rt.buffer("moe.delta", (T, self.hidden))
        if (x.dtype == torch.bfloat16 and T >= self.grouped_min_tokens
                and ops.moe_grouped_ok(self.hidden, self.ff, self.n_experts)):
            return self.forward_grouped(x, ids, weights, out)
        slices = ops.moe_rows_slices(self.ff)
        y = rt.buffer("moe.y", (T, self.top * slices, self.hidden), torch.float32)
        ops.moe_rows(x, self.w_gu, self.w_down, ids, y, self.limit, self.alpha)
        ops.moe_combine(y, weights, None, out, slices)
        return out

    def _library_grouped(self) -> bool:
        """Whether the two products of the sorted pairs go through the library's grouped product."""
        if os.environ.get("MLXFORGE_MOE_TILES", "0") == "1" or getattr(self.rt, "gemm_backend", "auto") == "tcgen05":
            return False
        return hasattr(torch, "_grouped_mm") and not torch.cuda.is_current_stream_capturing()

    def forward_grouped(self, x, ids, weights, out):
        """Many tokens: pairs ordered by expert, the two products over the sorted rows, the weighted sum in
        the order of the choice."""
        rt, T = self.rt, x.shape[0]
        i32, n = torch.int32, T * self.top
        slot_of = rt.buffer("moe.slot_of", (n,), i32)
        row_token = rt.buffer("moe.row_token", (n,), i32)
        meta = rt.buffer("moe.meta", (4,), i32)
        tiles = rt.buffer("moe.tiles", (3 * ops.moe_grouped_max_tiles(T, self.top, self.n_experts),), i32)
        ends = rt.buffer("moe.ends", (self.n_experts,), i32)
        ops.moe_sort(ids, self.n_experts, slot_of, row_token, meta, tiles, ends)
        act = rt.buffer("moe.act", (n, self.ff))
        if self._library_grouped():
            xg = rt.buffer("moe.xg", (n, self.hidden))
            ops.moe_gather_rows(x, row_token, xg)
            gu = torch._grouped_mm(xg, self.w_gu.view(self.n_experts, 2 * self.ff, self.hidden).transpose(1, 2), offs=ends)
            ops.moe_activation(gu, act, self.limit, self.alpha)
            y = torch._grouped_mm(act, self.w_down.transpose(1, 2), offs=ends)
            ops.moe_combine(y, weights, slot_of, out)
            return out
        ops.moe_grouped_up(x, self.w_gu, row_token, meta, tiles, act, self.top, self.limit, self.alpha)
        y = rt.buffer("moe.y", (n, self.hidden), torch.float32)
        ops.moe_grouped_down(act, self.w_down, meta, tiles, y, T, self.top)
        ops.moe_combine(y, weights, slot_of, out)
        return out
