"""A retention mixer: linear attention with one fixed decay per head and neither softmax nor denominator.  Per head a
matrix-valued state S [dk, dv] starts at zero and is carried from token to token:

    S <- decay_h S + k v^T;   o = S^T q

q and k pass a rotation by position (over all or the leading part of a head) and k is then multiplied by a scale; each
head's o is divided by its root mean square (no weight), multiplied by silu(W_g x), and leaves through the output product.
Options: `act="silu"` passes the projected q, k and v through silu first (the "lightning" form, which has no rotation and
no scale on k); `out_norm="all_heads"` norms all heads' results together as one vector with a stored weight over all of
them instead of head by head; `gate` is what the gate projection passes through (silu or sigmoid).

The products run on the engine's matrix kernels (q, k, v and the gate as one stacked product); the rotation, the
recurrence (csrc/retention.cu) and the output norm are kernels of their own and FP32 throughout.  Each request keeps S
(FP32) in its state slot, so a prompt may be cut anywhere and a decoded token costs one step of the recurrence.
"""
from __future__ import annotations

import torch

from .. import ops
from ..spec import PartSpec, TensorSpec
from . import linear
from .base import POSITION_ENCODINGS, Mixer, make_part, register_mixer, to_f32

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight", "o": "o_proj.weight", "norm": "norm.weight"}


@register_mixer("retention")
class Retention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_dim: int, decay, eps: float, pos: PartSpec, k_scale=None, names=None,
                 act=None, out_norm: str = "per_head", gate: str = "silu", norm_init: str = "ones"):
        """decay: one number per head.  k_scale: what k is multiplied by after the rotation (default head_dim^-1/2).
        act: None or "silu" on the projected q, k and v.  out_norm: "per_head" (no weight) or "all_heads" (one RMS norm over
        all heads' results with the stored weight `norm`).  gate: "silu" or "sigmoid"."""
        if act not in (None, "silu") or out_norm not in ("per_head", "all_heads") or gate not in ops.OUT_GATES:
            raise ValueError(f"retention: act {act!r}, out_norm {out_norm!r}, gate {gate!r}")
        self.act, self.out_norm, self.gate, self.norm_init = act, out_norm, gate, norm_init
        decay = [float(d) for d in decay]
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        self.D, self.H, self.dk, self.dv, self.decay, self.eps = hidden_size, num_heads, head_dim, v_dim, decay, float(eps)
        self.k_scale = float(k_scale) if k_scale is not None else head_dim ** -0.5
        self.pos = make_part(POSITION_ENCODINGS, "position encoding", pos)
        if not self.pos.is_identity and self.pos.rotary_dim > head_dim:
            raise ValueError(f"{self.pos.rotary_dim} turning dimensions in a head of {head_dim}")
        self.names = {**_NAMES, **(names or {})}
        # columns of the stacked product: [q | k | v | gate]
        self.k_col, self.v_col, self.g_col = num_heads * head_dim, 2 * num_heads * head_dim, 2 * num_heads * head_dim + num_heads * v_dim
        self.N = self.g_col + num_heads * v_dim

    def tensors(self):
        n, D, H, dk, dv = self.names, self.D, self.H, self.dk, self.dv
        out = [TensorSpec(n["q"], (H * dk, D)), TensorSpec(n["k"], (H * dk, D)), TensorSpec(n["v"], (H * dv, D)),
               TensorSpec(n["gate"], (H * dv, D)), TensorSpec(n["o"], (D, H * dv))]
        if self.out_norm == "all_heads":
            out.append(TensorSpec(n["norm"], (H * dv,), "f32", ("ones",) if self.norm_init == "ones" else ("ones_plus", 0.1)))
        return out

    def bind(self, get, rt):
        if self.dk > ops.retention_max_dim():
            raise ValueError(f"keys of {self.dk} entries: the retention kernel takes up to {ops.retention_max_dim()}")
        self.rt = rt
        n = self.names
        self.w_in = torch.empty((self.N, self.D), dtype=rt.dtype, device=rt.device)
        at = 0
        for name in ("q", "k", "v", "gate"):
            w = get(n[name])
            self.w_in[at:at + w.shape[0]].copy_(w)
            at += w.shape[0]
        self.w_o = torch.empty((self.D, self.H * self.dv), dtype=rt.dtype, device=rt.device)
        self.w_o.copy_(get(n["o"]))
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32).to(rt.device)
        # the output norm: per head without a weight, or one head of all heads' values with the stored weight
        self.out_w = to_f32(get(n["norm"]), rt) if self.out_norm == "all_heads" else torch.ones(self.dv, dtype=torch.float32, device=rt.device)
        self.pos.bind(lambda name: get("position." + name), rt)

    def state_shape(self):
        return {"S": ((self.H, self.dk, self.dv), torch.float32)}

    def forward(self, xn, ctx, cache, state, out):
        rt = self.rt
        ops.current_tag = "retention.in"
        p = linear.matmul(xn, self.w_in, rt)                                      # FP32 [T, q | k | v | gate]
        ops.current_tag = "retention.prepare"
        ops.retention_prep(p, self.H, self.dk, 0, self.k_col, None if self.pos.is_identity else self.pos.rotary_table(), self.k_scale,
                           ctx.positions, act_cols=self.g_col if self.act else 0)
        ops.current_tag = "retention.recurrence"
        o = ops.retention(p, 0, self.k_col, self.v_col, self.decay_t, state["S"], ctx.q_start, ctx.slot_ids, ctx.R, self.H, self.dk, self.dv)
        ops.current_tag = "retention.out"
        if self.out_norm == "all_heads":
            y = ops.delta_out(o, p, self.g_col, self.out_w, self.eps, 1, self.H * self.dv, rt.dtype, gate=self.gate)
        else:
            y = ops.delta_out(o, p, self.g_col, self.out_w, self.eps, self.H, self.dv, rt.dtype, gate=self.gate)
        ops.current_tag = "retention.o"
        return linear.matmul(y, self.w_o, rt, partials_ok=not ctx.hold_results)
