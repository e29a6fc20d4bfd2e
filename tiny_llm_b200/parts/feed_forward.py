"""SwiGLU feed-forward: m = (silu(y Wg^T) * (y Wu^T)) Wd^T, no biases
(tiny_llm/parser/llama_parser.cpp:225-249; tiny_llm/ops/cuda/silu.cu:7-12; arithmetic.cu:7-22).

The reference runs gate and up as two products over the same input, then SiLU, then the product.
Here the two weights are fused at load time into one matrix whose rows alternate in blocks of
`block` gate rows and `block` up rows, so that one output tile of the fused product holds matching
gate and up columns and SiLU * up can be taken in 32-bit where the accumulators are."""
from __future__ import annotations

import torch

from .. import ops
from ..weights import COMPUTE, WeightSpec
from .registry import register_part


def interleave_gate_up(wg: torch.Tensor, wu: torch.Tensor, block: int) -> torch.Tensor:
    """Rows [2 g block, 2 g block + block) are gate rows [g block, (g+1) block); the next `block`
    rows are the matching up rows.  `block` must divide the number of rows."""
    i, h = wg.shape
    assert i % block == 0
    g = i // block
    return torch.stack([wg.view(g, block, h), wu.view(g, block, h)], dim=1).reshape(2 * i, h).contiguous()


def scaled_matrix(w: torch.Tensor, scale: float) -> torch.Tensor:
    """`w` times a constant of the model, multiplied in 32-bit and rounded once to the matrix's own type."""
    if scale == 1.0:
        return w
    return (w.to(torch.float32) * scale).to(w.dtype).contiguous()


def gate_up_block(intermediate_size: int) -> int:
    for b in (128, 64, 32, 16, 8, 4, 2):
        if intermediate_size % b == 0:
            return b
    return 1


class SwiGLU:
    graph_safe = True   # launches kernels only: a step through this part can be captured in a CUDA graph

    def __init__(self, hidden_size: int, intermediate_size: int,
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight"), out_scale: float = 1.0,
                 act: str = "silu"):
        """`names`: what the gate, up and down matrices are called behind the part's prefix.  `out_scale`: a
        constant the part's output is multiplied by; it is folded into the down matrix when that is loaded.
        `act`: the gate's activation, "silu" or "relu" (m = (act(y Wg^T) * (y Wu^T)) Wd^T)."""
        if act not in ops.GLU_ACTS:
            raise ValueError(f"unknown gate activation {act!r}; known: {', '.join(ops.GLU_ACTS)}")
        self.act = act
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.names = tuple(names)
        self.out_scale = float(out_scale)
        self.block = gate_up_block(intermediate_size)
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self, prefix: str):
        i, h = self.intermediate_size, self.hidden_size
        g, u, d = self.names
        return [WeightSpec(prefix + g, (i, h), COMPUTE), WeightSpec(prefix + u, (i, h), COMPUTE),
                WeightSpec(prefix + d, (h, i), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        g, u, d = self.names
        self.w_gate_up = interleave_gate_up(weights[prefix + g], weights[prefix + u], self.block)
        self.w_down = scaled_matrix(weights[prefix + d], self.out_scale)

    def forward(self, ctx, h, resid) -> None:
        t = h.shape[0]
        act = ctx.workspace.get("ffn_act", (t, self.intermediate_size), ctx.dtype)
        ops.linear_swiglu(h, self.w_gate_up, act, self.block, ctx.workspace, act=self.act)
        ops.linear(act, self.w_down, resid, accumulate=True)


class DenseMLP:
    """Two matrices around an activation, no gate: m = Wd act(Wu y), act = relu(.)^2.  The first product leaves 32-bit
    sums; the activation is taken on them and rounded once."""
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, names=("up", "down"), act: str = "relu2",
                 out_scale: float = 1.0):
        if act not in ops.UNARY_ACTS or act == "copy":
            raise ValueError(f"unknown activation {act!r}; known: relu2")
        self.hidden_size, self.intermediate_size, self.names, self.act = hidden_size, intermediate_size, tuple(names), act
        self.out_scale = float(out_scale)
        self.w_up = self.w_down = None

    def weight_specs(self, prefix: str):
        u, d = self.names
        return [WeightSpec(prefix + u, (self.intermediate_size, self.hidden_size), COMPUTE),
                WeightSpec(prefix + d, (self.hidden_size, self.intermediate_size), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        u, d = self.names
        self.w_up = weights[prefix + u]
        self.w_down = scaled_matrix(weights[prefix + d], self.out_scale)

    def forward(self, ctx, h, resid) -> None:
        t = h.shape[0]
        sums = ctx.workspace.get("ffn_sums", (t, self.intermediate_size), torch.float32)
        ops.linear(h, self.w_up, sums)
        act = ctx.workspace.get("ffn_act", (t, self.intermediate_size), ctx.dtype)
        ops.unary(sums, act, self.act)
        ops.linear(act, self.w_down, resid, accumulate=True)


register_part("ffn", "swiglu", SwiGLU)
register_part("ffn", "dense_mlp", DenseMLP)
