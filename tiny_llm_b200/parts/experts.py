"""Mixture of experts: many small feed-forwards W_down act(W_up h), of which every token uses `top`.

Router: z = W_router h in 32-bit, s = sigmoid(z).  The experts with the largest s + correction are chosen (the
correction, one learned number per expert, steers the choice only); the chosen experts' outputs are summed with the
weights s * route_scale, not renormalised.  A shared expert of the same form runs for every token and is added times
sigmoid(w_sg . h), one number per token.  act is the exact (erf) GELU.

The experts' matrices are stacked at load ([experts, ff, hidden] and [experts, hidden, ff]); a step sorts its
(token, choice) pairs by expert into tiles of rows on the device, so that one grouped product serves all experts and
nothing about the routing reaches the host.  Prompt portions with enough rows per expert copy the grouped rows into
one contiguous matrix and run both products on the tcgen05 kernel (every tile of 128 rows reads its own expert's rows
of the stacked weights); smaller steps gather their rows inside an `mma.sync` (bfloat16) or FFMA (float32) kernel.  The router's rows and the shared gate's row are one matrix.

Variants, chosen by parameters.  `router="softmax"`: s = softmax(z) over all experts (the weights are still the chosen
experts' s * route_scale, not renormalised).  `correction=False`: the choice reads s alone and no correction tensor is
stored.  `glu="silu"` (or "relu"): an expert is W_down (act(W_gate h) * (W_up h)); its gate and up matrices are stacked
into one grouped product whose halves an element-wise kernel joins."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..weights import COMPUTE, FLOAT32, WeightSpec
from .feed_forward import scaled_matrix
from .registry import register_part


class RoutedExperts:
    graph_safe = True

    def __init__(self, hidden_size: int, num_experts: int, top: int, expert_size: int, route_scale: float = 1.0,
                 shared_size: Optional[int] = None, out_scale: float = 1.0, router: str = "sigmoid",
                 correction: bool = True, glu: Optional[str] = None):
        if not 0 < top <= num_experts:
            raise ValueError(f"{top} of {num_experts} experts cannot be chosen")
        if router not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router {router!r}; known: sigmoid, softmax")
        if glu is not None and glu not in ops.GLU_ACTS:
            raise ValueError(f"unknown gate activation {glu!r}; known: {', '.join(ops.GLU_ACTS)}")
        if glu is not None and shared_size is not None:
            raise ValueError("a shared expert beside gated experts is not built")
        self.router, self.has_correction, self.glu = router, correction, glu
        self.hidden_size, self.num_experts, self.top = hidden_size, num_experts, top
        self.expert_size, self.shared_size = expert_size, shared_size
        self.route_scale = float(route_scale)
        self.out_scale = float(out_scale)
        self.w_route = self.correction = self.w_up = self.w_down = self.w_shared_up = self.w_shared_down = None

    def weight_specs(self, prefix: str):
        h, f = self.hidden_size, self.expert_size
        specs = [WeightSpec(prefix + "router", (self.num_experts, h), COMPUTE)]
        if self.has_correction:
            specs.append(WeightSpec(prefix + "correction", (self.num_experts,), FLOAT32, init=("normal", 0.3)))
        for e in range(self.num_experts):
            if self.glu is not None:
                specs.append(WeightSpec(prefix + f"e{e}.gate", (f, h), COMPUTE))
            specs += [WeightSpec(prefix + f"e{e}.up", (f, h), COMPUTE), WeightSpec(prefix + f"e{e}.down", (h, f), COMPUTE)]
        if self.shared_size is not None:
            specs += [WeightSpec(prefix + "shared.up", (self.shared_size, h), COMPUTE),
                      WeightSpec(prefix + "shared.down", (h, self.shared_size), COMPUTE),
                      WeightSpec(prefix + "shared.sg", (1, h), COMPUTE)]
        return specs

    def load(self, prefix: str, weights) -> None:
        n = self.num_experts
        rows = [weights[prefix + "router"]] + ([weights[prefix + "shared.sg"]] if self.shared_size is not None else [])
        self.w_route = torch.cat(rows, dim=0).contiguous()
        self.correction = weights[prefix + "correction"] if self.has_correction else None
        if self.glu is not None:   # per expert [gate rows | up rows]: one grouped product gives both halves
            self.w_up = torch.stack([torch.cat([weights[prefix + f"e{e}.gate"], weights[prefix + f"e{e}.up"]], dim=0)
                                     for e in range(n)]).contiguous()
        else:
            self.w_up = torch.stack([weights[prefix + f"e{e}.up"] for e in range(n)]).contiguous()
        self.w_down = torch.stack([scaled_matrix(weights[prefix + f"e{e}.down"], self.out_scale) for e in range(n)]).contiguous()
        if self.shared_size is not None:
            self.w_shared_up = weights[prefix + "shared.up"]
            self.w_shared_down = scaled_matrix(weights[prefix + "shared.down"], self.out_scale)

    def forward(self, ctx, h, resid) -> None:
        t = h.shape[0]
        n, top, ws = self.num_experts, self.top, ctx.workspace
        logits = ws.get("moe_logits", (t, self.w_route.shape[0]), torch.float32)
        ops.linear(h, self.w_route, logits)
        ids = ws.get("moe_ids", (t, top), torch.int32)
        weights = ws.get("moe_weights", (t, top), torch.float32)
        ops.moe_route(logits, n, self.correction, self.route_scale, ids, weights, softmax=self.router == "softmax")
        pairs = t * top
        glu, f = self.glu, self.expert_size
        up_rows = 2 * f if glu is not None else f
        if ops.moe_tc_preferred(pairs, n, ctx.dtype, self.hidden_size, self.expert_size):
            # prompt portions: the rows of every expert as whole tiles of 128, made contiguous, through the tcgen05 product
            tile = ops.MOE_TC_TILE
            tiles = ops.moe_max_tiles(pairs, n, tile)
            sorted_rows = ws.get("moe_rows", (tiles * tile,), torch.int32)
            tile_expert = ws.get("moe_tile_expert", (tiles,), torch.int32)
            pair_pos = ws.get("moe_pair_pos", (pairs,), torch.int32)
            ops.moe_align(ids, n, tile, sorted_rows, tile_expert, pair_pos)
            grouped_in = ws.get("moe_in", (tiles * tile, self.hidden_size), ctx.dtype)
            ops.moe_gather(h, sorted_rows, tile_expert, tile, grouped_in, rows_per_input=top)
            act = ws.get("moe_act", (tiles * tile, f), ctx.dtype)
            if glu is not None:
                both = ws.get("moe_gate_up", (tiles * tile, up_rows), torch.float32)
                ops.moe_linear_tc(grouped_in, self.w_up, tile_expert, both)
                ops.silu_mul(both, act, f, act=glu)     # the product stores its sums: nothing to hand back zeroed
            else:
                ops.moe_linear_tc(grouped_in, self.w_up, tile_expert, act, gelu=True)
            y = ws.get("moe_y", (tiles * tile, self.hidden_size), torch.float32)
            ops.moe_linear_tc(act, self.w_down, tile_expert, y)
        else:
            pair_pos = None
            tile = ops.moe_tile_rows(pairs, n, tensor_cores=(ctx.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and
                                                             self.expert_size % 8 == 0))
            tiles = ops.moe_max_tiles(pairs, n, tile)
            sorted_rows = ws.get("moe_rows", (tiles * tile,), torch.int32)
            tile_expert = ws.get("moe_tile_expert", (tiles,), torch.int32)
            ops.moe_align(ids, n, tile, sorted_rows, tile_expert)
            act = ws.get("moe_act", (pairs, f), ctx.dtype)
            if glu is not None:
                both = ws.get("moe_gate_up", (pairs, up_rows), ctx.dtype)
                ops.moe_linear(h, self.w_up, sorted_rows, tile_expert, tile, both, rows_per_input=top, gelu=False)
                ops.silu_mul(both, act, f, act=glu)
            else:
                ops.moe_linear(h, self.w_up, sorted_rows, tile_expert, tile, act, rows_per_input=top, gelu=False if glu else True)
            y = ws.get("moe_y", (pairs, self.hidden_size), torch.float32)
            ops.moe_linear(act, self.w_down, sorted_rows, tile_expert, tile, y, rows_per_input=1, gelu=False)
        shared = None
        if self.shared_size is not None:
            sact = ws.get("ffn_act", (t, self.shared_size), ctx.dtype)
            ops.linear(h, self.w_shared_up, sact)
            ops.gelu(sact, sact)
            shared = ws.get("moe_shared", (t, self.hidden_size), torch.float32)
            ops.linear(sact, self.w_shared_down, shared)
        ops.moe_combine(y, weights, shared, logits, n, resid, pair_pos)


register_part("ffn", "routed_experts", RoutedExperts)
