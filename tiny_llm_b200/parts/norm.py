"""Norms.  RMSNorm: y_j = (w_j x_j) / sqrt(mean_j(x_j^2) + eps), statistics in 32-bit
(tiny_llm/ops/cuda/norm.cu:16-49).  Any width; the reference stops at 2048.  With `one_plus` the stored weight lies
around zero and the norm multiplies by 1 + w_j."""
from __future__ import annotations

from .. import ops
from ..weights import FLOAT32, WeightSpec
from .registry import register_part


class RMSNorm:
    graph_safe = True   # launches kernels only: a step through this part can be captured in a CUDA graph

    def __init__(self, size: int, eps: float, weight_suffix: str = ".weight", one_plus: bool = False,
                 scalar: bool = False):
        """`weight_suffix`: what the weight is called behind the part's name ("" when the name is the tensor's).
        `one_plus`: the norm multiplies by 1 + the stored weight (added once, in 32-bit, when the weight is loaded).
        `scalar`: the stored weight is ONE number for all coordinates (a tensor without dimensions); it is spread over
        the row when it is loaded."""
        self.size = size
        self.scalar = scalar
        self.eps = float(eps)
        self.weight_suffix = weight_suffix
        self.one_plus = one_plus
        self.weight = None

    def weight_specs(self, prefix: str):
        init = {"init": ("normal", 0.1)} if self.one_plus else ({"init": ("uniform", 0.5, 1.5)} if self.scalar else {})
        return [WeightSpec(prefix + self.weight_suffix, () if self.scalar else (self.size,), FLOAT32, **init)]

    def load(self, prefix: str, weights) -> None:
        w = weights[prefix + self.weight_suffix]
        if self.scalar:
            w = w.reshape(1).expand(self.size).contiguous()
        self.weight = (w + 1.0).contiguous() if self.one_plus else w

    def add_into(self, ctx, branch, resid, copy=None) -> None:
        """resid += norm(branch): for a block that norms a branch's output before it joins the stream.  `branch` is a
        zeroed float32 buffer that products added into; it is handed back zeroed.  `copy` (bfloat16) also receives the
        new stream, rounded."""
        ops.rms_norm_add(branch, self.weight, self.eps, 1.0, resid, copy=copy)

    def forward(self, ctx, x, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.workspace.get("norm_out", (n, self.size), ctx.dtype)
        ops.rms_norm(x, self.weight, self.eps, out, rows)
        return out


class DynamicTanh:
    """Dynamic Tanh: y_j = tanh(alpha x_j) w_j + b_j with one learned number alpha.  It takes the place of a norm and
    computes no mean or variance, so a row's output does not depend on the row's other values.  The weight is
    stored under the part's own name, the bias and alpha beside it as `<name>.b` and `<name>.alpha`."""
    graph_safe = True

    def __init__(self, size: int):
        self.size = size
        self.weight = self.bias = self.alpha = None

    def weight_specs(self, prefix: str):
        return [WeightSpec(prefix, (self.size,), FLOAT32),
                WeightSpec(prefix + ".b", (self.size,), FLOAT32, init=("normal", 0.05)),
                WeightSpec(prefix + ".alpha", (), FLOAT32, init=("const", 0.75))]

    def load(self, prefix: str, weights) -> None:
        self.weight = weights[prefix]
        self.bias = weights[prefix + ".b"]
        self.alpha = weights[prefix + ".alpha"].reshape(1).contiguous()

    def forward(self, ctx, x, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.workspace.get("norm_out", (n, self.size), ctx.dtype)
        ops.dyt_norm(x, self.weight, self.bias, self.alpha, out, rows)
        return out


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
