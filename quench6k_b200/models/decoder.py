"""The generic decoder: embedding, the executed list of blocks, final norm, LM head.

It is built from a spec.ModelSpec through the part registries and knows no architecture.  Tensor
names: `<embed_name>`, `<layer prefix>{input_layernorm,post_attention_layernorm}.*`,
`<layer prefix>self_attn.*` (the mixer's tensors), `<layer prefix>mlp.*` (the feed-forward's),
`<final_norm_prefix>*`, `<head_name>`.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from .. import ops
from ..parts import linear
from ..parts.base import (BLOCKS, EMBED_ADDS, FEED_FORWARDS, MIXERS, NORMS, CacheRequest, LayerCache, Runtime, WeightedRows, make_part,
                          to_operand)
from ..spec import ModelSpec, TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        D = spec.hidden_size
        self.blocks = []
        for ls in spec.layers:
            if ls.block not in BLOCKS:
                raise KeyError(f"unknown block arrangement {ls.block!r}; registered: {', '.join(sorted(BLOCKS))}")
            norm1 = make_part(NORMS, "norm", ls.norm, size=D)
            mixer = make_part(MIXERS, "mixer", ls.mixer, hidden_size=D)
            ffn = make_part(FEED_FORWARDS, "feed-forward", ls.ffn, hidden_size=D) if ls.ffn is not None else None
            norm2 = make_part(NORMS, "norm", ls.norm, size=D) if ffn is not None and not ls.shared_norm else None
            after = {}
            if ls.post_norm is not None:
                after["norm1b"] = make_part(NORMS, "norm", ls.post_norm, size=D)
                if ffn is not None:
                    after["norm2b"] = make_part(NORMS, "norm", ls.post_norm, size=D)
            if ls.side is not None:
                after["side"] = make_part(FEED_FORWARDS, "feed-forward", ls.side, hidden_size=D)
            self.blocks.append(BLOCKS[ls.block](norm1, mixer, norm2, ffn, **after, **ls.block_params))
        self.embed_norm = make_part(NORMS, "norm", spec.embed_norm, size=D) if spec.embed_norm is not None else None
        self.embed_add = make_part(EMBED_ADDS, "embedding add", spec.embed_add, hidden_size=D) if spec.embed_add is not None else None
        self.final_norm = make_part(NORMS, "norm", spec.final_norm, size=D)
        self.order = list(spec.order)
        self.kv_source = list(spec.kv_source)
        if len(self.kv_source) != len(self.order):
            raise ValueError("kv_source and order differ in length")
        self.readd = set(spec.readd_embedding)
        if any(not 0 < p < len(self.order) for p in self.readd):
            raise ValueError("readd_embedding names a position outside 1..executed layers - 1")
        self.rt: Optional[Runtime] = None

    # ------------------------------------------------------------------ declaration
    def tensors(self) -> List[TensorSpec]:
        s = self.spec
        out = [TensorSpec(s.embed_name, (s.vocab_size, s.hidden_size))]
        if self.embed_add is not None:
            out += [TensorSpec(s.embed_add_prefix + t.name, t.shape, t.role, t.init) for t in self.embed_add.tensors()]
        if self.embed_norm is not None:
            out += [TensorSpec(s.embed_norm_prefix + t.name, t.shape, t.role, t.init) for t in self.embed_norm.tensors()]
        if s.side_table is not None:
            out.append(TensorSpec(s.side_table[0], (s.vocab_size, s.side_table[1])))
        for ls, b in zip(s.layers, self.blocks):
            for sub, part in b.parts():
                out += [TensorSpec(ls.prefix + s.sub_names[sub] + t.name, t.shape, t.role, t.init) for t in part.tensors()]
        out += [TensorSpec(s.final_norm_prefix + t.name, t.shape, t.role, t.init) for t in self.final_norm.tensors()]
        if s.head_name is not None:
            out.append(TensorSpec(s.head_name, (s.vocab_size, s.hidden_size)))
        return out

    def cache_requests(self) -> List[Optional[CacheRequest]]:
        """Per executed position: the cache its mixer needs (None for positions that borrow one
        or whose mixer keeps no keys)."""
        out = []
        for p, i in enumerate(self.order):
            out.append(None if self.kv_source[p] is not None else self.blocks[i].mixer.cache_request())
        return out

    def state_shapes(self):
        """Per executed position: the shape of its mixer's fixed-size per-request state, or None; one more entry, the state of
        what the model adds to its embedding output, if it has such a part."""
        return [self.blocks[i].mixer.state_shape() for i in self.order] + ([self.embed_add.state_shape()] if self.embed_add is not None else [])

    def graph_safe(self) -> bool:
        parts = [self.final_norm] + [x for x in (self.embed_norm, self.embed_add) if x is not None]
        for b in self.blocks:
            parts += [part for _, part in b.parts()]
        return all(getattr(x, "graph_safe", False) for x in parts)

    # ------------------------------------------------------------------ weights
    def bind(self, get: Callable[[str], torch.Tensor], rt: Runtime) -> None:
        s = self.spec
        self.rt = rt
        self.embed = to_operand(get(s.embed_name), rt)
        if self.embed_add is not None:
            self.embed_add.bind(lambda n: get(s.embed_add_prefix + n), rt)
        if self.embed_norm is not None:
            self.embed_norm.bind(lambda n: get(s.embed_norm_prefix + n), rt)
        self.side_table = to_operand(get(s.side_table[0]), rt) if s.side_table is not None else None
        for ls, b in zip(s.layers, self.blocks):
            for sub, part in b.parts():
                pre = ls.prefix + s.sub_names[sub]
                part.bind(lambda n, pre=pre: get(pre + n), rt)
        self.final_norm.bind(lambda n: get(s.final_norm_prefix + n), rt)
        self.head = self.embed if s.head_name is None else to_operand(get(s.head_name), rt)

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, caches: List[Optional[LayerCache]], states: List[Optional[torch.Tensor]]) -> Optional[torch.Tensor]:
        """Runs the tokens of `ctx` through the executed layers; returns FP32 logits
        [len(ctx.logit_rows), vocab] or None when no row is wanted."""
        ops.current_tag = "embedding"
        h = ops.embed(ctx.token_ids, self.embed, fed=ctx.fed)
        if self.embed_add is not None:
            ops.current_tag = "embedding.add"
            self.embed_add.forward(h, ctx, states[len(self.order)])
        if self.embed_norm is not None:
            ops.current_tag = "norm.embedding"
            self.embed_norm.normalize(h)
        if self.side_table is not None:
            ops.current_tag = "embedding.side"
            ctx.side_rows = ops.embed(ctx.token_ids, self.side_table, fed=ctx.fed)
        h0 = h.clone() if self.readd else None      # the embedding output, for the passes of a repeated span that take it again
        pending = None                      # an add into h that a block has left to the next norm
        for p, i in enumerate(self.order):
            ctx.position = p
            block = self.blocks[i]
            if p in self.readd:
                if block.takes_extra:
                    pending = block.forward(h, ctx, caches[p], states[p], pending, extra=h0)
                    continue
                if pending is not None:
                    pending.apply(h)
                    pending = None
                h += h0
            pending = block.forward(h, ctx, caches[p], states[p], pending)
        if ctx.n_logit_rows == 0:
            return None
        # an add that is left: the last norm makes it if it can (it normalises picked rows only, so a sublayer result that
        # passes a norm of its own is added first, for all rows)
        if pending is not None and not (isinstance(pending, WeightedRows) and self.final_norm.fuses_weighted_rows):
            pending.apply(h)
            pending = None
        ops.current_tag = "norm.final"
        xn = self.final_norm.forward(h, rows=ctx.logit_rows, add=pending)
        ops.current_tag = "lm_head"
        return linear.matmul(xn, self.head, self.rt)
