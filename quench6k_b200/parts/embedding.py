"""What a model may add to its embedding output before the first layer.

"token_pair": a second table indexed by a hash of the token and the one before it,

    h[t] += table[(token[t-1] * mul_prev + token[t] * mul_cur) mod buckets],    h[first] += table[buckets]

(the table has buckets + 1 rows; the last one serves a sequence's first token, which has no token before it).  The token
before a portion's first row is per-request state: one int32 in the request's state slot, which every step leaves at the
portion's last token, so a prompt may be cut anywhere and a decoded token finds its predecessor there.
"""
from __future__ import annotations

import torch

from .. import ops
from ..spec import TensorSpec
from .base import EmbedAdd, register_embed_add, to_operand


@register_embed_add("token_pair")
class TokenPairEmbedding(EmbedAdd):
    graph_safe = True

    def __init__(self, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, name: str = "weight"):
        if buckets < 1 or mul_prev < 0 or mul_cur < 0:
            raise ValueError(f"token pairs: {buckets} buckets, multipliers {mul_prev} and {mul_cur}")
        self.D, self.buckets, self.mul_prev, self.mul_cur, self.name = hidden_size, int(buckets), int(mul_prev), int(mul_cur), name

    def tensors(self):
        return [TensorSpec(self.name, (self.buckets + 1, self.D))]

    def bind(self, get, rt):
        self.rt = rt
        self.table = to_operand(get(self.name), rt)

    def state_shape(self):
        return {"prev": ((), torch.int32)}

    def forward(self, h, ctx, state):
        ops.embed_pair(h, ctx.token_ids, self.table, self.mul_prev, self.mul_cur, ctx.positions, ctx.req_of_token, ctx.q_start, ctx.slot_ids,
                       state["prev"], fed=ctx.fed)
