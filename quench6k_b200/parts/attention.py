"""Grouped-query self-attention over the paged cache, with optional per-head QK-norm, learned
sinks and a sliding window (reference: crates/engine/src/flint.rs:815-913 for the order of
operations, crates/cuda/kernels/flint.cu:125-173 and :211-561 for the arithmetic).

Beyond the reference: values of another width than the keys (v_dim), a given score scale, a mask of chunks (a position
sees the earlier positions of its own block of `chunk` positions, blocks counted from position 0), and the heads'
softmax weights mixed by a learned [heads, heads] matrix before they meet the values (`talk`).  Layers that use any of
these run the flexible attention kernels; the others run as before.  Two more options change what enters the attention,
not the attention: biases on the q, k and v projections, and a short causal convolution over time on every channel of
the projected q, k and v (before normalisation and rotation), whose last taps - 1 inputs are kept per request in a state
slot so that a prompt may be cut anywhere.

Further options, each a parameter: a bias on the output projection (`o_bias`); a sink of a fixed score instead of learned
ones (`fixed_sink`: a sink of 0 adds one to every softmax denominator); q/k norms without stored weights
(`qk_norm_weight=False`: the vectors are divided by their root mean square, which commutes with the rotation); values that
are the key projection's raw results (`values_are_keys`: no value projection is stored and the
stacked product has q and k only; the kernels that write the pages store the key, as it stands before its norm, as the
value); a cap on the scaled scores
(`softcap`: s -> c tanh(s / c)); and difference attention (`maps=2` with `diff`): every head attends twice, with queries
and keys of its own per map (q and k hold a head's maps side by side, the q/k norm weights are shared by all heads and
maps) over the same values, and the head's result is o = a1 - L a2 divided by its root mean square over the value
width, times (1 - diff), where L = exp(lq1 . lk1) - exp(lq2 . lk2) + diff is one number made from four stored vectors."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..spec import PartSpec, TensorSpec
from . import linear
from .base import (POSITION_ENCODINGS, CacheRequest, Mixer, make_part, register_mixer, to_f32, to_operand)


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, eps: float,
                 pos: PartSpec, window: Optional[int] = None, sinks: bool = False, qk_norm: bool = False,
                 norm_init: str = "ones", sink_std: float = 1.0, v_dim: Optional[int] = None, scale: Optional[float] = None,
                 chunk: Optional[int] = None, talk: bool = False, names=None, bias: bool = False, conv: Optional[int] = None,
                 o_bias: bool = False, fixed_sink: Optional[float] = None, qk_norm_weight: bool = True, values_are_keys: bool = False,
                 softcap: Optional[float] = None, maps: int = 1, diff: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        self.D, self.Hq, self.Hkv, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.vd = int(v_dim) if v_dim else head_dim
        self.eps, self.window, self.has_sinks, self.qk_norm = float(eps), window, sinks, qk_norm
        self.chunk, self.talk = (int(chunk) if chunk else None), bool(talk)
        self.norm_init, self.sink_std = norm_init, sink_std
        self.pos = make_part(POSITION_ENCODINGS, "position encoding", pos)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        # the flexible kernels: any widths, chunks, mixed heads; the fixed-shape kernels: everything the reference has
        self.has_o_bias, self.fixed_sink, self.qk_norm_weight = bool(o_bias), fixed_sink, bool(qk_norm_weight)
        self.values_are_keys, self.softcap, self.maps = bool(values_are_keys), float(softcap or 0.0), int(maps)
        self.diff = float(diff) if diff is not None else None
        if self.maps not in (1, 2) or (self.maps == 2) != (self.diff is not None):
            raise ValueError(f"{maps} maps with diff {diff!r}: difference attention has two maps and a diff, plain attention one and none")
        if sinks and fixed_sink is not None:
            raise ValueError("learned sinks and a fixed sink exclude each other")
        if self.values_are_keys and (self.vd != head_dim or self.maps > 1 or conv):
            raise ValueError("values that are the keys have the keys' width, one map and no convolution")
        if self.values_are_keys and self.pos.rotary_table() is None and not self.pos.is_identity:
            raise ValueError("values that are the keys take a rotation of pairs or no position encoding")
        if self.talk and (sinks or fixed_sink is not None or self.maps > 1 or self.softcap):
            raise ValueError("mixed heads are combined with neither sinks, maps nor a cap on the scores")
        self.flexible = (self.vd != head_dim or self.chunk is not None or self.talk or self.maps > 1 or self.softcap > 0.0
                         or head_dim % 16 != 0 or head_dim > 256)
        self.has_bias, self.taps = bool(bias), (int(conv) if conv else 0)
        if self.taps > 16:
            raise ValueError(f"{self.taps} convolution taps: the kernel takes 1 to 16")
        if self.flexible and self.pos.rotary_table() is None and not self.pos.is_identity:
            raise ValueError("the flexible attention kernels take a rotation of pairs or no position encoding")
        if self.talk and (num_heads > 64 or self.vd > 256):
            raise ValueError(f"mixed heads: at most 64 heads and values up to 256 wide, not {num_heads} and {self.vd}")
        if not self.flexible and (head_dim % 16 or head_dim > 256):
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 up to 256")
        # the tensors' names relative to the part's prefix (an architecture may call them anything)
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "q_norm": "q_norm.weight",
                      "k_norm": "k_norm.weight", "sinks": "sinks", "talk": "talk.weight", "q_bias": "q_proj.bias", "k_bias": "k_proj.bias",
                      "v_bias": "v_proj.bias", "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight",
                      "o_bias": "o_proj.bias", "lq1": "lambda_q1", "lk1": "lambda_k1", "lq2": "lambda_q2", "lk2": "lambda_k2", **(names or {})}
        # rows of the stacked projection: a head's maps side by side in q and k, one value head per KV head
        self.nq, self.nk = num_heads * self.maps * head_dim, num_kv_heads * self.maps * head_dim
        self.nv = 0 if self.values_are_keys else num_kv_heads * self.vd

    def tensors(self):
        D, Hq, Hkv, hd, n = self.D, self.Hq, self.Hkv, self.hd, self.names
        out = [TensorSpec(n["q"], (self.nq, D)), TensorSpec(n["k"], (self.nk, D))]
        if not self.values_are_keys:
            out.append(TensorSpec(n["v"], (self.nv, D)))
        out.append(TensorSpec(n["o"], (D, Hq * self.vd)))
        if self.qk_norm and self.qk_norm_weight:
            init = ("ones",) if self.norm_init == "ones" else ("ones_plus", 0.1)
            out += [TensorSpec(n["q_norm"], (hd,), "f32", init), TensorSpec(n["k_norm"], (hd,), "f32", init)]
        if self.has_sinks:
            out.append(TensorSpec(n["sinks"], (Hq,), "f32", ("normal", self.sink_std)))
        if self.talk:
            out.append(TensorSpec(n["talk"], (Hq, Hq), "f32", ("normal", 0.5)))
        widths = (("q", self.nq), ("k", self.nk), ("v", self.nv))
        if self.has_bias:
            out += [TensorSpec(n[x + "_bias"], (c,), "f32", ("normal", 0.1)) for x, c in widths if not (x == "v" and self.values_are_keys)]
        if self.has_o_bias:
            out.append(TensorSpec(n["o_bias"], (D,), "f32", ("normal", 0.1)))
        if self.maps > 1:
            out += [TensorSpec(n[x], (hd,), "f32", ("normal", 0.1)) for x in ("lq1", "lk1", "lq2", "lk2")]
        if self.taps:
            out += [TensorSpec(n[x + "_conv"], (c, self.taps), "f32", ("normal", 0.5)) for x, c in widths]
        out += [TensorSpec("position." + t.name, t.shape, t.role, t.init) for t in self.pos.tensors()]
        return out

    def bind(self, get, rt):
        self.rt = rt
        # q, k and v rows stacked so one product yields [q | k | v] per token: each piece is copied into its place
        # on the device as it arrives, so that no two copies of the three are held at once
        nq, nk, nv, n = self.nq, self.nk, self.nv, self.names
        pieces = ("q", "k") if self.values_are_keys else ("q", "k", "v")
        self.w_qkv = torch.empty((nq + nk + nv, self.D), dtype=rt.dtype, device=rt.device)
        for name, lo, hi in ((n["q"], 0, nq), (n["k"], nq, nq + nk), (n["v"], nq + nk, nq + nk + nv))[:len(pieces)]:
            self.w_qkv[lo:hi].copy_(get(name))
        self.w_q = self.w_qkv[:nq]
        self.w_o = to_operand(get(n["o"]), rt)
        if self.qk_norm and self.qk_norm_weight:
            self.q_norm, self.k_norm = to_f32(get(n["q_norm"]), rt), to_f32(get(n["k_norm"]), rt)
        elif self.qk_norm:
            self.q_norm = self.k_norm = torch.ones(self.hd, dtype=torch.float32, device=rt.device)
        else:
            self.q_norm = self.k_norm = None
        self.sinks = to_f32(get(n["sinks"]), rt) if self.has_sinks else None
        if self.fixed_sink is not None:
            self.sinks = torch.full((self.Hq,), float(self.fixed_sink), dtype=torch.float32, device=rt.device)
        self.w_talk = to_f32(get(n["talk"]), rt) if self.talk else None
        # biases and taps of q, k and v side by side, like the rows of the stacked product
        self.bias = torch.cat([to_f32(get(n[x + "_bias"]), rt) for x in pieces]).contiguous() if self.has_bias else None
        # biases without a convolution are added by the kernel that normalises q and k and writes the pages (an encoding that
        # is no rotation of pairs has no such kernel in front of it: its biases take the convolution kernel with one tap)
        self.prep_bias = self.bias if self.has_bias and not self.taps and (self.flexible or self.pos.rotary_table() is not None or self.pos.is_identity) else None
        if self.has_o_bias:
            self.o_bias = to_f32(get(n["o_bias"]), rt)
            self._one_tap = torch.ones((self.D, 1), dtype=torch.float32, device=rt.device)
            self._no_o_tail = torch.zeros((1, 0, self.D), dtype=torch.float32, device=rt.device)
        if self.maps > 1:
            lq1, lk1, lq2, lk2 = (get(n[x]).to(torch.float32).cpu() for x in ("lq1", "lk1", "lq2", "lk2"))
            # FP32 throughout, as a model holds it: two dot products, two exponentials, one difference
            self.map_weight = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + torch.tensor(self.diff, dtype=torch.float32))
        self.conv_w = torch.cat([to_f32(get(n[x + "_conv"]), rt) for x in "qkv"]).contiguous() if self.taps else None
        if self.has_bias and not self.taps and self.prep_bias is None:          # a bias alone: one tap of weight one
            self.conv_w = torch.ones((nq + nk + nv, 1), dtype=torch.float32, device=rt.device)
        self._no_tail = torch.zeros((1, 0, nq + nk + nv), dtype=torch.float32, device=rt.device)
        self.pos.bind(lambda name: get("position." + name), rt)

    def cache_request(self):
        v = self.vd if self.vd != self.hd else None
        heads = {"kv_heads": self.Hkv * self.maps, "v_heads": self.Hkv if self.maps > 1 else None}     # a key head per map, one value head
        if self.chunk is not None and (self.window is None or self.window >= self.chunk):
            return CacheRequest("chunked", self.chunk, head_dim=self.hd, v_dim=v, **heads)      # what a chunk's start hides, no later query sees
        if self.window is not None:
            return CacheRequest("sliding", int(self.window), head_dim=self.hd, v_dim=v, **heads)
        return CacheRequest("full", None, head_dim=self.hd, v_dim=v, **heads)

    def state_shape(self):
        if self.taps > 1:
            return {"conv": ((self.taps - 1, self.nq + self.nk + self.nv), torch.float32)}
        return None

    def _after_projection(self, qkv, ctx, cache, state):
        """Bias and short convolution on the projected q, k and v (FP32, possibly split-K partial sums): FP32 [T, q | k | v]."""
        if self.conv_w is None:
            return qkv
        if not cache.write:
            raise ValueError("a layer that borrows another's keys cannot convolve its own")
        ops.current_tag = "attention.conv"
        tail = state["conv"] if self.taps > 1 else self._no_tail
        return ops.short_conv(qkv, self.conv_w.shape[0], self.conv_w, self.bias, tail, ctx.req_of_token, ctx.q_start, ctx.slot_ids, ctx.R)

    def _forward_flexible(self, xn, ctx, cache, state=None):
        """Any key and value widths, a window and/or chunks, mixed heads: the flexible kernels."""
        rt, write = self.rt, cache.write
        table = ctx.block_tables[cache.group]
        ops.current_tag = "attention.qkv"
        qkv = self._after_projection(linear.matmul(xn, self.w_qkv if write else self.w_q, rt, partials_ok=True), ctx, cache, state)
        ops.current_tag = "attention.prepare"
        M = self.maps
        q = ops.qkv_pages(qkv, self.Hq * M, self.Hkv * M, self.hd, self.vd, self.q_norm, self.k_norm, self.eps, self.pos.rotary_table(),
                          ctx.positions, ctx.req_of_token, table if write else None, cache.page_size, cache.k if write else None,
                          cache.v if write else None, rt.dtype, v_heads=self.Hkv, bias=self.prep_bias, values_are_keys=self.values_are_keys)
        ops.current_tag = "attention.keys"
        tiles = None if rt.is_fp32 or not rt.tensor_cores else ctx.query_tiles(ops.attention_flex_tile_tokens(self.Hq, self.Hkv))
        a = ops.attention_flex(None, q.view(-1, self.hd), False, cache.k, cache.v, table, ctx.req_of_token, ctx.positions, self.Hq * M,
                               self.scale, window=self.window, chunk=self.chunk, talk=self.w_talk, tiles=tiles, max_context=ctx.max_context,
                               sinks=self.sinks, softcap=self.softcap, maps=M, out_f32=M > 1)
        if M > 1:                                   # a head's two maps, FP32, into the head's one result
            ops.current_tag = "attention.maps"
            a = ops.map_difference(a, self.Hq, self.vd, self.map_weight, self.eps, 1.0 - self.diff, rt.dtype)
        ops.current_tag = "attention.o"
        return self._out(a, ctx)

    def _out(self, a, ctx):
        """The output projection (FP32, possibly split-K slices) and its bias."""
        rt = self.rt
        if not self.has_o_bias or ctx.leave_bias:
            if self.has_o_bias:
                ctx.left_bias = self.o_bias                       # the block adds it together with the result
            return linear.matmul(a, self.w_o, rt, partials_ok=not ctx.hold_results)
        y = linear.matmul(a, self.w_o, rt, partials_ok=True)
        ops.current_tag = "attention.o_bias"                      # the slices summed and the bias added: one tap of weight one
        return ops.short_conv(y, self.D, self._one_tap, self.o_bias, self._no_o_tail, ctx.req_of_token, ctx.q_start, ctx.slot_ids, ctx.R)

    def forward(self, xn, ctx, cache, state, out):
        if self.flexible:
            return self._forward_flexible(xn, ctx, cache, state)
        rt = self.rt
        write = cache.write
        # which attention kernels this step takes, and the plan of the key splits, before anything of the layer is
        # launched: the kernel that splits the keys reads its plan while the kernel before it still runs
        ops.current_tag = "attention.plan"
        how = self._choose(cache, ctx)
        rotary = self.pos.rotary_table()
        fused_pos = rotary is not None or self.pos.is_identity
        # a step of a few tokens per request: the kernel that splits the keys normalises and rotates q itself and makes
        # the new keys and values (one launch less)
        in_attention = (self.prepare_in_attention and how[0] == "split" and fused_pos and self.conv_w is None and self.prep_bias is None and
                        not self.values_are_keys and
                        ops.attention_mma_prepares(self.hd, self.Hq // self.Hkv, how[1][0], rotary[1] if rotary else 0, bool(rotary and rotary[2])))
        # FP32 [T, (Hq + 2 Hkv) hd] or [T, Hq hd]; for few rows possibly as split-K partials, which the next kernel sums
        ops.current_tag = "attention.qkv"
        qkv = self._after_projection(linear.matmul(xn, self.w_qkv if write else self.w_q, rt, partials_ok=fused_pos), ctx, cache, state)
        table = ctx.block_tables[cache.group]
        if in_attention:
            ops.current_tag = "attention.keys"
            a = self._split_keys(None, cache, table, ctx, how[1],
                                 prepare={"qkv": qkv, "heads": self.Hq, "q_norm": self.q_norm, "k_norm": self.k_norm, "eps": self.eps,
                                          "rotary": rotary, "write": write})
            ops.current_tag = "attention.o"
            return self._out(a, ctx)
        ops.current_tag = "attention.prepare"
        if not fused_pos:
            qkv = self._unfused_position(qkv, ctx, write)
            q = ops.qk_prep(qkv, self.Hq, self.Hkv, self.hd, None, None, self.eps, None, ctx.positions, ctx.req_of_token,
                            table if write else None, cache.page_size, cache.k if write else None,
                            cache.v if write else None, rt.dtype)
        else:
            q = ops.qk_prep(qkv, self.Hq, self.Hkv, self.hd, self.q_norm, self.k_norm, self.eps, rotary, ctx.positions,
                            ctx.req_of_token, table if write else None, cache.page_size, cache.k if write else None,
                            cache.v if write else None, rt.dtype, bias=self.prep_bias, values_are_keys=self.values_are_keys)
        ops.current_tag = "attention.keys"
        a = self._attend(q, cache, table, ctx, how)
        # the block adds it into the stream inside its next norm (which also sums split-K partials)
        ops.current_tag = "attention.o"
        return self._out(a, ctx)

    prepare_in_attention = True   # the kernel that splits the keys makes q and the new keys itself where it can (else qk_prep does)
    tc_min_fill = 0.5             # the tcgen05 prompt kernel runs when its CTAs (two tiles each) cover at least this share of the SMs

    def _choose(self, cache, ctx):
        """("generic",) | ("split", plan args) | ("tc", tile pairs, plan args of the short requests or None): the tensor-core
        kernels for bfloat16 where they cover the head and group size, else the generic one.  The plans are made here."""
        rt, G = self.rt, self.Hq // self.Hkv
        rows = 0 if rt.is_fp32 or not rt.tensor_cores else ops.attention_mma_tile_rows(self.hd, G, ctx.max_q_len)
        if not rows:
            return ("generic",)
        if rows > 16 and ops.attention_tc_supported(self.hd, G, cache.page_size):
            tile = ops.attention_tc_tile_tokens(G)
            # beside prompt portions, requests with a few tokens (decoded tokens, the stub of a prompt) go to the kernel
            # that splits the keys over CTAs: as a tile of their own they would walk their whole context in one CTA
            cut = tile // 2 if ctx.R > 1 else 0
            tok0, ntok, n_pairs = ctx.query_tile_pairs(tile, zigzag=False, more_than=cut)
            if n_pairs * self.Hkv >= self.tc_min_fill * self._sm_count():
                # prompt portions with enough tiles (two to a CTA) to fill that share of the SMs: both products on tcgen05, no key splits
                count, _, _, most, _ = ctx.short_requests(cut)
                short = self._plan(ctx, ops.attention_mma_tile_rows(self.hd, G, most), cut) if count else None
                return ("tc", (tok0, ntok), short)
        return ("split", self._plan(ctx, rows, None))

    def _plan(self, ctx, rows, at_most):
        """The tiles and the plan of the key splits for the mma.sync kernel over all requests of the step, or over those
        with at most `at_most` tokens.  The keys are split over one wave of resident CTAs, and no further (a second,
        partly filled wave would cost as much as a full one); the plan is made on the device, once per step for all
        layers with this window."""
        tokens = rows // (self.Hq // self.Hkv)
        tok0, ntok, n_tiles = ctx.query_tiles(tokens, at_most)
        key = ("attention_plan", tokens, at_most, self.window, self.Hkv)
        fresh = key not in ctx.made
        if fresh:                                   # the first layer of this pass with these tiles and this window
            ctx.plans[key] = ops.attention_plan(ctx.positions, ctx.req_of_token, tok0, ntok, self.window,
                                                ops.attention_mma_resident_ctas(self.hd, rows) // self.Hkv, min_per=2,
                                                into=ctx.plans.get(key))
            ctx.made.add(key)
        return rows, tok0, ntok, ctx.plans[key], fresh

    def _attend(self, q, cache, table, ctx, how):
        if how[0] == "generic":
            return ops.attention_generic(q, cache.k, cache.v, table, ctx.req_of_token, ctx.positions, self.window, self.sinks, self.scale)
        if how[0] == "tc":
            (tok0, ntok), short = how[1], how[2]
            out = ops.attention_tc(q, cache.k, cache.v, table, ctx.req_of_token, ctx.positions, tok0, ntok, self.window,
                                   self.sinks, scale=self.scale)
            return out if short is None else self._split_keys(q, cache, table, ctx, short, out)
        return self._split_keys(q, cache, table, ctx, how[1])

    def _split_keys(self, q, cache, table, ctx, planned, out=None, prepare=None):
        rows, tok0, ntok, plan, fresh = planned
        # The plan was made before this layer's first launch.  With q from qk_prep, the kernel before this one is that
        # one (or, beside prompt portions, the tcgen05 attention), which itself waited for everything before it: the plan
        # is complete when this kernel starts.  When this kernel prepares q itself, the kernel before it is the q/k/v
        # product, which may itself have started before the one before it ended: then only a plan of an earlier layer
        # is surely complete.
        return ops.attention_mma(q, cache.k, cache.v, table, ctx.req_of_token, ctx.positions, tok0, ntok, rows, self.window,
                                 self.sinks, scale=self.scale, out=out, plan=plan, plan_is_old=prepare is None or not fresh,
                                 prepare=prepare)

    def _sm_count(self) -> int:
        if "_sms" not in self.__dict__:
            self._sms = torch.cuda.get_device_properties(self.rt.device).multi_processor_count
        return self._sms

    def _unfused_position(self, qkv, ctx, write):
        """QK-norm, then a position encoding that is no rotation of pairs (its own `apply`), on FP32 q and k."""
        T = qkv.shape[0]
        nq, nk = self.Hq * self.hd, self.Hkv * self.hd
        q = qkv[:, :nq].reshape(T * self.Hq, self.hd).contiguous()
        if self.qk_norm:
            q = ops.rmsnorm(q, self.q_norm, self.eps, torch.float32)
        q = q.view(T, self.Hq, self.hd)
        self.pos.apply(q, ctx.positions)
        parts = [q.reshape(T, nq)]
        if write:
            k = qkv[:, nq:nq + nk].reshape(T * self.Hkv, self.hd).contiguous()
            if self.qk_norm:
                k = ops.rmsnorm(k, self.k_norm, self.eps, torch.float32)
            k = k.view(T, self.Hkv, self.hd)
            self.pos.apply(k, ctx.positions)
            parts += [k.reshape(T, nk), qkv[:, nq + nk:]]
        return torch.cat(parts, dim=1).contiguous()
