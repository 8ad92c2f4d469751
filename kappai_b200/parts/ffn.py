"""SwiGLU feed-forward.

``f = (silu(h Wg^T) * (h Wu^T)) Wd^T`` added to the residual; gate and up run
as one product against [Wg; Wu], gate rows first (src/recipe/builders.c:344-388,
src/model.c:1575-1610); ``silu(g) = g / (1 + exp(-g))``
(src/backend/cpu/quants.h:369-371).

Params: hidden_size, intermediate_size, bias, activation (``silu`` by default;
``relu`` and ``gelu_tanh`` make the same unit with another function on the gate:
kind ``glu``).

``moe``: a mixture of ``num_experts`` such units without biases, of which every
row uses the ``top`` with the largest router logits ``z = h Wr^T + b`` (float32),
weighted by the softmax over those ``top`` logits alone; see csrc/moe.cu.
Params: hidden_size, expert_size, num_experts, top, activation, router_bias.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels as K
from ..ops.linear import linear, linear_swiglu
from ..config.schema import ConfigError
from .base import Part, WeightSpec, register_part


class SwiGLU(Part):
    category = "feed_forward"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.ff = int(self._p("intermediate_size"))
        self.bias = bool(self._p("bias", False))
        self.activation = str(self._p("activation", "silu"))
        K.activation_code(self.activation)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {"gate_proj.weight": WeightSpec((self.ff, self.d)), "up_proj.weight": WeightSpec((self.ff, self.d)),
             "down_proj.weight": WeightSpec((self.d, self.ff))}
        if self.bias:
            s["gate_proj.bias"] = WeightSpec((self.ff,), "bias")
            s["up_proj.bias"] = WeightSpec((self.ff,), "bias")
            s["down_proj.bias"] = WeightSpec((self.d,), "bias")
        return s

    def bind(self, w):
        self.w_gu = torch.cat([w["gate_proj.weight"], w["up_proj.weight"]], 0).contiguous()
        self.w_down = w["down_proj.weight"].contiguous()
        self.b_gu = self.b_down = None
        if self.bias:
            self.b_gu = torch.cat([w["gate_proj.bias"].float(), w["up_proj.bias"].float()]).contiguous()
            self.b_down = w["down_proj.bias"].float().contiguous()

    def forward(self, h, residual, ctx):
        act = linear_swiglu(h, self.w_gu, self.b_gu, self.activation)
        linear(act, self.w_down, self.b_down, out=residual, accumulate=True)


class MixtureOfExperts(Part):
    category = "feed_forward"
    graph_safe = True          # rows meet their experts on the device; the host sees none of it

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.ff = int(self._p("expert_size"))
        self.E = int(self._p("num_experts"))
        self.top = int(self._p("top"))
        self.activation = str(self._p("activation", "silu"))
        self.router_bias = bool(self._p("router_bias", True))
        K.activation_code(self.activation)
        if self.E < 1 or not (1 <= self.top <= self.E):
            raise ConfigError(f"moe: top={self.top} must lie between 1 and num_experts={self.E}")
        if self.top > K.MOE_MAX_TOP or self.E > K.MOE_MAX_EXPERTS:
            raise ConfigError(f"moe: the kernels take top <= {K.MOE_MAX_TOP} and num_experts <= {K.MOE_MAX_EXPERTS}")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {"router.weight": WeightSpec((self.E, self.d))}
        if self.router_bias:
            s["router.bias"] = WeightSpec((self.E,), "bias")
        for e in range(self.E):
            s[f"experts.{e}.gate_proj.weight"] = WeightSpec((self.ff, self.d))
            s[f"experts.{e}.up_proj.weight"] = WeightSpec((self.ff, self.d))
            s[f"experts.{e}.down_proj.weight"] = WeightSpec((self.d, self.ff))
        return s

    def bind(self, w):
        # the router is 32-bit whatever the storage of the rest
        self.w_router = w["router.weight"].to(torch.float32).contiguous()
        self.b_router = w["router.bias"].to(torch.float32).contiguous() if self.router_bias else None
        self.w_gu = torch.stack([torch.cat([w[f"experts.{e}.gate_proj.weight"], w[f"experts.{e}.up_proj.weight"]], 0)
                                 for e in range(self.E)]).contiguous()                       # [E, 2 ff, d]
        self.w_down = torch.stack([w[f"experts.{e}.down_proj.weight"] for e in range(self.E)]).contiguous()   # [E, d, ff]

    def forward(self, h, residual, ctx):
        n = h.shape[0]
        idx = torch.empty((n, self.top), dtype=torch.int32, device=h.device)
        weights = torch.empty((n, self.top), dtype=torch.float32, device=h.device)
        layout = torch.empty(K.moe_layout_ints(n, self.E, self.top), dtype=torch.int32, device=h.device)
        if K.moe_router_ok(self.d, self.E) and h.stride(1) == 1:
            K.moe_router(h, self.w_router, self.b_router, self.top, idx, weights, layout)
        else:
            logits = linear(h, self.w_router, self.b_router, out_dtype=torch.float32)
            K.moe_route(logits, self.top, idx, weights, layout)
        K.moe_experts(h, self.w_gu, self.w_down, layout, weights, self.top, residual, self.activation)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "glu", SwiGLU)
register_part("feed_forward", "moe", MixtureOfExperts)
