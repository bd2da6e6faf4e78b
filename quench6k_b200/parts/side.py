"""A per-layer token input: a small sublayer whose gate is multiplied by an embedding of the token itself.

The model holds one side table [vocab, layers * dim]; every layer owns `dim` columns of it.  With e the token's row of
those columns and x the stream:

    g = gelu_tanh(W_gate x) * e;     y = W_proj g

The block that holds the part adds y to the stream through the part's own RMS norm (a plain weight, `norm`).  The step
gathers the tokens' rows of the table once (`StepContext.side_rows`, FP32 [T, layers * dim]) and every layer reads its
columns.
"""
from __future__ import annotations

from .. import ops
from ..spec import TensorSpec
from . import linear
from .base import FeedForward, register_feed_forward, to_operand
from .norm import RMSNorm


@register_feed_forward("token_side")
class TokenSide(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, dim: int, column: int, eps: float, names=None, norm_init: str = "ones"):
        """column: the first of this layer's `dim` columns in the step's side rows."""
        self.D, self.dim, self.column = hidden_size, int(dim), int(column)
        self.names = {"gate": "gate_proj.weight", "proj": "proj.weight", "norm": "norm.weight", **(names or {})}
        self.norm = RMSNorm(hidden_size, eps, init=norm_init, weight_name=self.names["norm"])

    def tensors(self):
        n = self.names
        return [TensorSpec(n["gate"], (self.dim, self.D)), TensorSpec(n["proj"], (self.D, self.dim))] + self.norm.tensors()

    def bind(self, get, rt):
        self.rt = rt
        self.w_gate, self.w_proj = to_operand(get(self.names["gate"]), rt), to_operand(get(self.names["proj"]), rt)
        self.norm.bind(get, rt)

    def compute(self, x, ctx):
        """y, FP32 [T, D] (or split-K slices of it)."""
        if ctx.side_rows is None:
            raise ValueError("the step carries no side rows: the model has no side table")
        ops.current_tag = "side.gate"
        p = linear.matmul(x, self.w_gate, self.rt, partials_ok=True)
        g = ops.side_gate(p, ctx.side_rows, self.column, self.rt.dtype)
        ops.current_tag = "side.proj"
        return linear.matmul(g, self.w_proj, self.rt, partials_ok=True)

    def forward(self, x, ctx, out):
        self.norm.add_normed(out, self.compute(x, ctx))
