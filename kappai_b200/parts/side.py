"""Parts that act on the residual itself, outside the mixer and the feed-forward.

``token_gated`` (category ``side``): a per-layer token input at the end of a
layer.  With ``e`` the columns ``[part * dim, (part + 1) * dim)`` of a second
token table's row for the row's token,

    g = act(x Wgate^T) * e ;  y = g Wproj^T ;  x <- x + y / sqrt(mean(y^2) + eps) * w

(act = tanh-gelu).  It reads the residual ``x`` (in the compute type), not a
normed copy.  The table belongs to the model (kind ``token_table``) and is
handed to the part after loading (``attach``).

``concat_linear`` (category ``entry``): ``x <- W [x; x0]`` with ``W``
[hidden, 2 hidden], the columns of ``x`` first: the residual mixed with the
embedding output ``x0`` at the head of a pass over a stretch of layers.  It runs
as two products, one over each half of ``W``; the second adds into the first's
float32 output.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.schema import ConfigError
from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, register_part


def compute_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 rows ``x`` as a matrix operand of the compute type (``x`` itself in 32-bit)."""
    if dtype == torch.float32:
        return x
    return K.cast(x, torch.empty(x.shape, dtype=dtype, device=x.device))


class TokenGatedInput(Part):
    category = "side"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.dim = int(self._p("dim"))
        self.part = int(self._p("part"))
        self.eps = float(self._p("eps"))
        self.activation = str(self._p("activation", "gelu_tanh"))
        K.activation_code(self.activation)
        if self.dim < 1 or self.part < 0:
            raise ConfigError("token_gated: dim must be positive and part must not be negative")
        self.table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"gate.weight": WeightSpec((self.dim, self.d)), "proj.weight": WeightSpec((self.d, self.dim)),
                "norm.weight": WeightSpec((self.d,), "norm")}

    def bind(self, w):
        self.w_gate = w["gate.weight"].contiguous()
        self.w_proj = w["proj.weight"].contiguous()
        self.norm_w = w["norm.weight"].float().contiguous()

    def attach(self, table_part) -> None:
        if (self.part + 1) * self.dim > table_part.width:
            raise ConfigError(f"token_gated: part {self.part} of {self.dim} columns lies outside the table's {table_part.width}")
        self.table = table_part.weight

    def forward(self, x, ctx):
        gate = linear(compute_rows(x, self.env.dtype), self.w_gate)
        g = K.token_gate(gate, self.table, self.part * self.dim, ctx.token_ids, torch.empty_like(gate), self.activation)
        y = linear(g, self.w_proj, out_dtype=torch.float32)
        K.rmsnorm_add_rows(y, self.norm_w, self.eps, x)


class ConcatLinearEntry(Part):
    category = "entry"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.d, 2 * self.d))}

    def bind(self, w):
        self.w_x = w["weight"][:, :self.d].contiguous()
        self.w_x0 = w["weight"][:, self.d:].contiguous()

    def forward(self, x, h0):
        """``x``: the float32 residual; ``h0``: the embedding output in the compute type.  Returns the new residual."""
        out = torch.empty_like(x)
        linear(compute_rows(x, self.env.dtype), self.w_x, out=out)
        linear(h0, self.w_x0, out=out, accumulate=True)
        return out


register_part("side", "token_gated", TokenGatedInput)
register_part("entry", "concat_linear", ConcatLinearEntry)
