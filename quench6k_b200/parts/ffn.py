"""Feed-forward parts: a dense SwiGLU MLP and a routed mixture of SwiGLU experts with an optional
ungated shared expert.

Reference: crates/engine/src/flint.rs:915-1075 (order of operations),
crates/cuda/kernels/flint.cu:829-868 (sigmoid routing), crates/cuda/kernels/moe.cu:19-71 (softmax
routing), flint.cu:1163-1239 (permutation, SwiGLU, combine in slot order).  The reference runs
its dense MLP and its shared expert as extra expert slots with weight 1; here they are the dense
part, added after the routed sum.
"""
from __future__ import annotations


import torch

from .. import ops
from ..spec import TensorSpec
from . import linear
from .base import FeedForward, WeightedRows, register_feed_forward, to_f32, to_operand


def _checked_act(act):
    if isinstance(act, (tuple, list)):
        if len(act) != 2 or act[0] not in ops.GATES_WITH_LIMIT:
            raise ValueError(f"unknown gate {act!r}; with a constant: {', '.join(ops.GATES_WITH_LIMIT)}")
        return (act[0], float(act[1]))
    if act not in ops.ACTIVATIONS:
        raise ValueError(f"unknown activation {act!r}; known: {', '.join(ops.ACTIVATIONS)}")
    return act


@register_feed_forward("dense")
class DenseSwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, names=None, act: str = "silu"):
        """act: what the gate passes through, one of ops.ACTIVATIONS, or a gate with its constant such as ("clamped", limit)
        (ops.GATES_WITH_LIMIT); applied in the epilogue of the gate/up product."""
        self.D, self.I, self.act = hidden_size, intermediate_size, _checked_act(act)
        # the tensors' names relative to the part's prefix (an architecture may call them anything)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight", **(names or {})}

    def tensors(self):
        n = self.names
        return [TensorSpec(n["gate"], (self.I, self.D)), TensorSpec(n["up"], (self.I, self.D)), TensorSpec(n["down"], (self.D, self.I))]

    def bind(self, get, rt):
        self.rt = rt
        self.w_gate, self.w_up = to_operand(get(self.names["gate"]), rt), to_operand(get(self.names["up"]), rt)
        self.w_down = to_operand(get(self.names["down"]), rt)

    def _gated(self, xn):
        ops.current_tag = "dense.gate_up"
        return linear.swiglu_matmul(xn, self.w_gate, self.w_up, self.rt, act=None if self.act == "silu" else self.act)

    def forward(self, xn, ctx, out):
        act = self._gated(xn)
        ops.current_tag = "dense.down"
        linear.matmul(act, self.w_down, self.rt, out=out, accumulate=True)

    def compute(self, xn, ctx):
        """The result itself, FP32 [T, D] (or split-K slices of it), for a block whose norm takes it before the stream does."""
        act = self._gated(xn)
        ops.current_tag = "dense.down"
        return linear.matmul(act, self.w_down, self.rt, partials_ok=True)


@register_feed_forward("moe")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, intermediate_size: int, scoring: str = "softmax",
                 renormalize: bool = True, shared_intermediate_size: int = 0, gated: bool = True, act: str = "silu",
                 correction: bool = False, route_scale: float = 1.0, names=None, shared_act=None, shared_prefix: str = "shared_experts.",
                 shared_names=None, groups=None):
        """gated: an expert is down(act(gate x) * (up x)); else down(act(up x)).  correction: a stored vector added to the
        scores for the choice of the experts only (the weights use the scores without it); route_scale multiplies the
        weights.  groups = (count, keep): the experts form `count` equal groups of neighbours, and only experts of the `keep`
        groups whose two largest choice values add up to most can be chosen.  All three belong to sigmoid scoring (with
        renormalised weights, or with the plain scores as weights).  act may be a gate with its constant, such as
        ("clamped", limit) (gated experts only).  The shared expert has the experts' form with an activation (shared_act,
        default the experts'), a tensor prefix and tensor names of its own."""
        act = _checked_act(act)
        if isinstance(act, tuple) and not gated:
            raise ValueError(f"the gate {act[0]!r} belongs to gated experts")
        self.gated, self.act, self.has_correction, self.route_scale = bool(gated), act, bool(correction), float(route_scale)
        self.groups = (int(groups[0]), int(groups[1])) if groups is not None and int(groups[0]) > 1 else None
        if self.groups is not None and (num_experts % self.groups[0] or not 0 < self.groups[1] <= self.groups[0]
                                        or top_k > self.groups[1] * (num_experts // self.groups[0])):
            raise ValueError(f"{num_experts} experts in {self.groups[0]} groups of which {self.groups[1]} are kept, {top_k} chosen")
        self.own_router = self.has_correction or self.route_scale != 1.0 or self.groups is not None
        if self.own_router and scoring != "sigmoid":
            raise ValueError("a correction of the choice, groups of experts and a scale of the weights go with sigmoid scores")
        self.names = {"router": "gate.weight", "gate": "experts.gate_proj.weight", "up": "experts.up_proj.weight",
                      "down": "experts.down_proj.weight", "correction": "gate.correction", **(names or {})}
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown router scoring {scoring!r}")
        if not 0 < top_k <= num_experts:
            raise ValueError(f"top_k {top_k} outside 1..{num_experts}")
        self.D, self.E, self.k, self.I = hidden_size, num_experts, top_k, intermediate_size
        self.scoring, self.renorm = scoring, bool(renormalize)
        self.shared_prefix = shared_prefix
        self.shared = (DenseSwiGLU(hidden_size, shared_intermediate_size, names=shared_names, act=shared_act if shared_act is not None else act)
                       if shared_intermediate_size > 0 else None)
        self.always_defers = self.shared is None      # forward(defer=True) never touches `out`
        self.pair_tokens = 16                         # steps of at most this many tokens run the experts pair by pair
        self.routing_tap = None               # a parts.base.Tap: every forward records each row's chosen experts [T, k]
                                              # ("experts") and its router logits [T, E] ("router_logits") there

    def tensors(self):
        E, I, D, n = self.E, self.I, self.D, self.names
        out = [TensorSpec(n["router"], (E, D))]
        if self.gated:
            out.append(TensorSpec(n["gate"], (E, I, D)))
        out += [TensorSpec(n["up"], (E, I, D)), TensorSpec(n["down"], (E, D, I))]
        if self.has_correction:
            out.append(TensorSpec(n["correction"], (E,), "f32", ("normal", 0.1)))
        if self.shared is not None:
            out += [TensorSpec(self.shared_prefix + t.name, t.shape, t.role, t.init) for t in self.shared.tensors()]
        return out

    def bind(self, get, rt):
        self.rt = rt
        n = self.names
        self.w_router = to_operand(get(n["router"]), rt)
        self.w_up = to_operand(get(n["up"]), rt)
        self.w_gate = to_operand(get(n["gate"]), rt) if self.gated else self.w_up      # ungated: the first (only) product's weights
        self.w_down = to_operand(get(n["down"]), rt)
        self.correction = to_f32(get(n["correction"]), rt) if self.has_correction else None
        if self.shared is not None:
            self.shared.bind(lambda n: get(self.shared_prefix + n), rt)

    defers_add = True

    def _tap(self, ctx, sel_e, logits):
        if logits.dim() == 3:                 # split-K slices of the router product: summed in order, as the routing kernel sums them
            total = logits[0].clone()
            for s in range(1, logits.shape[0]):
                total += logits[s]
            logits = total
        self.routing_tap.record("experts", ctx.position, sel_e)
        self.routing_tap.record("router_logits", ctx.position, logits)

    def compute(self, xn, ctx):
        """(the shared expert's result FP32 [T, D] or split-K slices of it, or None; the routed experts' results unsummed,
        a WeightedRows): for a block whose norm takes the sum before the stream does."""
        rows = self.forward(xn, ctx, None, defer=True, routed_only=True)
        return (self.shared.compute(xn, ctx) if self.shared is not None else None), rows

    def forward(self, xn, ctx, out, defer=False, routed_only=False):
        """Adds the experts' weighted results into `out`; with defer=True and no shared expert it
        returns them unsummed (WeightedRows) for the next norm to add.  routed_only: the shared expert is the caller's."""
        rt = self.rt
        T = xn.shape[0]
        pairs = T * self.k
        defer = defer and (self.shared is None or routed_only)
        if (self.gated and self.act == "silu" and not self.own_router and rt.tensor_cores and not rt.is_fp32 and ops.router_small_supported(T, self.E, self.D, self.k)
                and ops.tc_supported(xn, self.w_gate) and self.I % 8 == 0):
            # a decode step: router and top-k in one launch, then one weight tile stream per
            # (token, slot) pair straight from the selection, no permutation and no gather
            ops.current_tag = "experts.router"
            sel_e, sel_w, order, logits = ops.router_small(xn, self.w_router, self.k, self.scoring, self.renorm, with_logits=True)
            if self.routing_tap is not None:
                self._tap(ctx, sel_e, logits)
            ops.current_tag = "experts.gate_up"
            if ops.gemv_preferred(T, self.I, self.D):                     # a token or two: the matrix-vector kernel per pair
                act = ops.gemv(xn, self.w_gate, w2=self.w_up, pair_expert=sel_e.view(-1), pair_div=self.k)
                ops.current_tag = "experts.down"
                y = ops.gemv(act, self.w_down, pair_expert=sel_e.view(-1), pair_div=1, pairs_are_old=True)   # the router made them, two kernels ago
            else:
                act = ops.gemm_tc_pairs(xn, self.w_gate, sel_e, self.k, w2=self.w_up, order=order)  # [pairs, I]
                ops.current_tag = "experts.down"
                y = ops.gemm_tc_pairs(act, self.w_down, sel_e, 1, order=order, pairs_are_old=True)   # FP32 [pairs, D]
            if defer:
                return WeightedRows(y, sel_w)
            ops.current_tag = "experts.combine"
            ops.combine(y, None, sel_w, out)
            if self.shared is not None:
                self.shared.forward(xn, ctx, out)
            return None
        ops.current_tag = "experts.router"
        logits = linear.matmul(xn, self.w_router, rt, partials_ok=True)    # FP32 [T, E], or split-K slices of it that route() sums
        if self.own_router:
            sel_e, sel_w = ops.route_biased(logits, self.k, self.correction, self.route_scale, renorm=self.renorm, groups=self.groups)
        else:
            sel_e, sel_w = ops.route(logits, self.k, self.scoring, self.renorm)
        if self.routing_tap is not None:
            self._tap(ctx, sel_e, logits)
        if (T <= self.pair_tokens and defer and rt.tensor_cores and not rt.is_fp32 and ops.tc_supported(xn, self.w_up) and self.I % 8 == 0):
            # a step of a few tokens whose router is not the one-launch kernel's: still one weight tile stream per
            # (token, slot) pair straight from the selection, no permutation and no gather
            ops.current_tag = "experts.gate_up"
            act = self.act if not self.gated or self.act != "silu" else None
            first = ops.gemm_tc_pairs(xn, self.w_gate, sel_e, self.k, w2=self.w_up if self.gated else None, act=act)     # [pairs, I]
            ops.current_tag = "experts.down"
            return WeightedRows(ops.gemm_tc_pairs(first, self.w_down, sel_e, 1, pairs_are_old=True), sel_w)
        ops.current_tag = "experts.permute"
        plan = linear.group_plan(xn, self.w_gate, sel_e, rt)             # permutation by expert, row tiles, gathered rows
        ops.current_tag = "experts.gate_up"
        if self.gated:
            act = linear.grouped_swiglu(xn, plan, self.w_gate, self.w_up, rt, act=None if self.act == "silu" else self.act)   # [pairs, I]
        else:
            act = linear.grouped_activated(xn, plan, self.w_up, rt, self.act)
        ops.current_tag = "experts.down"
        y = linear.grouped_matmul(act, plan, self.w_down, rt)                                     # FP32 [pairs, D]
        if defer:
            return WeightedRows(y, sel_w, plan.pair_row)
        ops.current_tag = "experts.combine"
        ops.combine(y, plan.pair_row, sel_w, out)
        if self.shared is not None:
            self.shared.forward(xn, ctx, out)
        return None
