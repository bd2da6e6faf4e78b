"""RMSNorm with a plain weight: out = x * rsqrt(mean(x^2) + eps) * w, computed in FP32
(reference: crates/cuda/kernels/flint.cu:97-122), and layer norm with weight and bias."""
from __future__ import annotations

from .. import ops
from ..spec import TensorSpec
from .base import Norm, PostNormed, WeightedRows, register_norm, to_f32


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, init: str = "ones", weight_name: str = "weight", offset: float = 0.0):
        """offset: the stored weight is the multiplier minus this (1.0: a weight kept around zero); the sum is made once, in
        FP32, when the weight is bound.  weight_name: the tensor's name relative to the norm's prefix."""
        self.size, self.eps, self.init = size, float(eps), init
        self.weight_name, self.offset = weight_name, float(offset)

    def tensors(self):
        init = {"ones": ("ones",), "zeros": ("normal", 0.0)}.get(self.init, ("normal", 0.1) if self.offset else ("ones_plus", 0.1))
        return [TensorSpec(self.weight_name, (self.size,), "f32", init)]

    def bind(self, get, rt):
        self.rt = rt
        self.weight = to_f32(get(self.weight_name), rt)
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    fuses_weighted_rows = True

    def add_normed(self, h, y, weighted=None, out_dtype=None):
        """h += this norm of (y + weighted rows) in place (y FP32 [T, D] or [slices, T, D] partial sums, or None; weighted a
        WeightedRows or None); with out_dtype also the stream as it then stands, in that dtype."""
        w = None if weighted is None else (weighted.y, weighted.pair_row, weighted.weights)
        return ops.add_normed(h, y, self.weight, self.eps, out_dtype, weighted=w)

    def normalize(self, h):
        """h <- this norm of h, in place on the FP32 stream."""
        return ops.rmsnorm(h, self.weight, self.eps, h.dtype, out=h)

    def forward(self, h, rows=None, add=None):
        if isinstance(add, WeightedRows):
            return ops.rmsnorm(h, self.weight, self.eps, self.rt.dtype, rows=rows, weighted=(add.y, add.pair_row, add.weights))
        return ops.rmsnorm(h, self.weight, self.eps, self.rt.dtype, rows=rows, add=add)


@register_norm("layernorm")
class LayerNorm(Norm):
    """out = (x - mean) / sqrt(var + eps) * w + b, the variance being the mean of the squared deviations; FP32.
    weight_name / bias_name: the tensors' names relative to the norm's prefix (an architecture may call them anything)."""
    graph_safe = True
    fuses_post_normed = True

    def __init__(self, size: int, eps: float, init: str = "ones", weight_name: str = "weight", bias_name: str = "bias"):
        self.size, self.eps, self.init = size, float(eps), init
        self.weight_name, self.bias_name = weight_name, bias_name

    def tensors(self):
        plain = self.init == "ones"
        return [TensorSpec(self.weight_name, (self.size,), "f32", ("ones",) if plain else ("ones_plus", 0.1)),
                TensorSpec(self.bias_name, (self.size,), "f32", ("normal", 0.0 if plain else 0.1))]

    def bind(self, get, rt):
        self.rt = rt
        self.weight, self.bias = to_f32(get(self.weight_name), rt), to_f32(get(self.bias_name), rt)

    def add_normed(self, h, y):
        ops.layernorm(h, None, None, self.eps, self.rt.dtype, after=(y, self.weight, self.bias))

    def forward(self, h, rows=None, add=None, extra=None):
        """add: a PostNormed of a layer norm (h += its norm of its y, in the same pass), or FP32 to be added as it is;
        extra: FP32 of h's shape, added after that."""
        after = None
        if isinstance(add, PostNormed) and isinstance(add.norm, LayerNorm) and add.norm.eps == self.eps and rows is None:
            after = (add.y, add.norm.weight, add.norm.bias)
        elif add is not None:
            if hasattr(add, "apply"):
                add.apply(h)
            else:
                h += add if add.dim() == 2 else add.sum(0)
        if rows is not None and extra is not None:
            h += extra
            extra = None
        return ops.layernorm(h, self.weight, self.bias, self.eps, self.rt.dtype, rows=rows, after=after, extra=extra)
