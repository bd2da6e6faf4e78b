"""Attention over a cached latent: per token one low-rank vector c (RMS-normed) and one rotated key part shared by all
heads are cached; a head's key is [W_uk_h c | rotated part], its value W_uv_h c.  Scores and output are computed in the
latent space, which needs nothing but the cache: with q_h = [a_h | r_h],

    score_h(i, j) = scale * ((W_uk_h^T a_h(i)) . c(j) + r_h(i) . k_rot(j)),     out_h(i) = W_uv_h (sum_j p_h(i, j) c(j)),

so every head attends with a query of rank + rot_dim over one shared key row per position whose first `rank` entries
are also its value: multi-query attention over the pages, between two per-head products.

Options: a sliding window (position i sees j with 0 <= i - j < window), a learned sink per head (exp(sink_h) joins the
softmax denominator), either pairing of the rotation, and a layer that has no down-projection of its own but reads the
pages another layer wrote (`borrows`: its own queries, up-projections, mask and output product).  A layer whose pages
are read by layers with wider windows keeps them for the widest (`retain`: a window, or None for every key)."""
from __future__ import annotations

from .. import ops
from ..spec import PartSpec, TensorSpec
from . import linear
from .base import POSITION_ENCODINGS, CacheRequest, Mixer, make_part, register_mixer, to_f32, to_operand

_NAMES = {"q": "q_proj.weight", "dkv": "kv_down_proj.weight", "c_norm": "kv_norm.weight", "uk": "k_up_proj.weight",
          "uv": "v_up_proj.weight", "out": "o_proj.weight", "sinks": "sinks"}


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_dim: int, kv_rank: int, scale: float, eps: float,
                 pos: PartSpec, names=None, norm_init: str = "ones", window=None, sinks: bool = False, sink_std: float = 1.0,
                 borrows: bool = False, retain="window"):
        """window: the sliding window's size (None: causal).  sinks: a learned number per head in the softmax denominator.
        borrows: no down-projection and no pages of its own (the model names the layer whose pages it reads).  retain:
        how long this layer's pages are kept: "window" (its own window), an integer (a wider window of a layer that
        reads them) or None (every key)."""
        self.D, self.H, self.dim, self.rd, self.vd, self.rank = hidden_size, num_heads, head_dim, rot_dim, v_dim, kv_rank
        self.scale, self.eps, self.norm_init = float(scale), float(eps), norm_init
        if kv_rank > 512:
            raise ValueError(f"a latent of {kv_rank}: the attention kernels take values up to 512 wide")
        self.pos = make_part(POSITION_ENCODINGS, "position encoding", pos)
        if not self.pos.is_identity and self.pos.rotary_dim > rot_dim:
            raise ValueError("the rotated part turns over at most rot_dim dimensions")
        self.window = int(window) if window else None
        self.has_sinks, self.sink_std, self.borrows = bool(sinks), sink_std, bool(borrows)
        self.retain = self.window if retain == "window" else (int(retain) if retain else None)
        if self.window is not None and self.retain is not None and self.retain < self.window:
            raise ValueError(f"pages kept for {self.retain} positions under a window of {self.window}")
        self.names = {**_NAMES, **(names or {})}

    def tensors(self):
        n, H = self.names, self.H
        init = ("ones",) if self.norm_init == "ones" else ("ones_plus", 0.1)
        out = [TensorSpec(n["q"], (H * (self.dim + self.rd), self.D))]
        if not self.borrows:
            out += [TensorSpec(n["dkv"], (self.rank + self.rd, self.D)), TensorSpec(n["c_norm"], (self.rank,), "f32", init)]
        out += [TensorSpec(n["uk"], (H * self.dim, self.rank)), TensorSpec(n["uv"], (H * self.vd, self.rank))]
        if self.has_sinks:
            out.append(TensorSpec(n["sinks"], (H,), "f32", ("normal", self.sink_std)))
        return out + [TensorSpec(n["out"], (self.D, H * self.vd))]

    def bind(self, get, rt):
        import torch
        self.rt = rt
        n, H = self.names, self.H
        nq = H * (self.dim + self.rd)
        own = 0 if self.borrows else self.rank + self.rd
        self.w_qd = torch.empty((nq + own, self.D), dtype=rt.dtype, device=rt.device)     # one product: [q | latent | shared key part]
        self.w_qd[:nq].copy_(get(n["q"]))
        if not self.borrows:
            self.w_qd[nq:].copy_(get(n["dkv"]))
        self.c_norm = None if self.borrows else to_f32(get(n["c_norm"]), rt)
        self.sinks = to_f32(get(n["sinks"]), rt) if self.has_sinks else None
        # per head: a -> W_uk_h^T a is a product with the [rank, dim] matrix W_uk_h^T; o -> W_uv_h o with [vd, rank]
        self.w_ukT = to_operand(get(n["uk"]), rt).view(H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = to_operand(get(n["uv"]), rt).view(H, self.vd, self.rank).contiguous()
        self.w_o = to_operand(get(n["out"]), rt)
        self.pos.bind(lambda name: get("position." + name), rt)

    def cache_request(self):
        if self.borrows:
            return None
        if self.retain is not None:
            return CacheRequest("sliding", self.retain, 1, self.rank + self.rd, v_dim=self.rank, values_in_keys=True)
        return CacheRequest("full", None, 1, self.rank + self.rd, v_dim=self.rank, values_in_keys=True)

    def forward(self, xn, ctx, cache, state, out):
        rt, H = self.rt, self.H
        T = xn.shape[0]
        if cache is None or cache.write == self.borrows:
            raise ValueError("a latent attention layer writes its own pages unless it borrows another layer's, and then only reads")
        table = ctx.block_tables[cache.group]
        ops.current_tag = "latent.qkv"
        x = linear.matmul(xn, self.w_qd, rt)
        ops.current_tag = "latent.prepare"
        inv_freq, turn, neighbours = (None, 0, False) if self.pos.is_identity else self.pos.rotary_table()
        qn, qr = ops.latent_prep(x, H, self.dim, self.rd, self.rank, self.c_norm, self.eps, inv_freq, turn, ctx.positions,
                                 ctx.req_of_token, table, cache.page_size, cache.k, neighbours=neighbours, write=not self.borrows)
        ops.current_tag = "latent.absorb"
        ql = linear.batched_matmul(qn.view(H * T, self.dim), self.w_ukT, rt, T)          # FP32 [H T, rank]
        ops.current_tag = "latent.keys"
        tiles = None if rt.is_fp32 or not rt.tensor_cores else ctx.query_tiles(ops.attention_flex_tile_tokens(H, 1))
        o = ops.attention_flex(ql, qr.view(H * T, self.rd) if self.rd else None, True, cache.k, cache.v, table, ctx.req_of_token,
                               ctx.positions, H, self.scale, window=self.window, out_head_major=True, tiles=tiles,
                               max_context=ctx.max_context, sinks=self.sinks)                                       # [H, T, rank]
        ops.current_tag = "latent.values"
        ov = linear.batched_matmul(o.view(H * T, self.rank), self.w_uv, rt, T)           # FP32 [H T, vd]
        a = ops.heads_to_rows(ov, H, rt.dtype)
        ops.current_tag = "latent.o"
        return linear.matmul(a, self.w_o, rt, partials_ok=True)
