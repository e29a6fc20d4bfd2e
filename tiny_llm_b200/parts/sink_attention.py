"""Softmax attention with a sink and an output gate, in two forms.

Both share the softmax: beside the visible keys' terms its denominator holds exp(sink_h), a learned score per head
that stands for no key and has no value, so a head may give weight to nothing.  Both multiply the heads' outputs by
sigmoid(Wg h) of the mixer's own input before the output projection.  Scores, the softmax, norms, angles and the
gate's sigmoid are 32-bit; the attention kernel leaves float32 rows and the gate kernel rounds them once.

`SinkAttention`: grouped-query heads with optional biases on q, k, v, optional norms of every query and key head
(x / sqrt(mean(x^2) + eps) * w, one weight vector of the key size for all heads), no rotation, and optionally a query
that grows with the logarithm of its position, q <- q (1 + coef ln(floor((p + 1) / every) + 1)).  Key size and value
size may differ.  The gate has one value per output value.

`LatentAttention`: keys and values of all heads are projections of ONE small latent vector per token,
    c = norm(first `rank` rows of Wdkv h),   k_h = [Wuk_h c | rot(last rows of Wdkv h)],   v_h = Wuv_h c,
and the queries are [plain | rotated] per head.  Only c and the rotated key part are cached.  The scores are taken
against the cache as it is: with q'_h = Wuk_h^T q_plain_h the score q_plain_h . (Wuk_h c) equals q'_h . c, so every
head attends with the query [q'_h | q_rot_h] over one shared key row [c | k_rot] and one shared value row c, and the
head's value projection is applied to the weighted sum of latents afterwards: o_h = Wuv_h (sum_j p_j c_j).  The rotated
parts turn in pairs (2i, 2i + 1) by p * base^(-2i / rot_dims).  A key is visible while 0 <= i - j < window.  The gate
has one value per head."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache import KVNeed
from ..weights import COMPUTE, FLOAT32, WeightSpec
from .feed_forward import scaled_matrix
from .registry import register_part


def pair_frequencies(dims: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2: computed in 64-bit, kept in 32-bit."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(torch.float32).contiguous()


def _padded(n: int) -> int:
    return -(-n // 8) * 8


class SinkAttention:
    graph_safe = True   # launches kernels only

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 eps: float, bias: bool = True, qk_norm: bool = True, sink: bool = True, gate: bool = True,
                 stretch_coef: float = 0.0, stretch_every: int = 0, window: Optional[int] = None,
                 out_scale: float = 1.0, shares_cache: bool = False):
        if shares_cache:
            raise ValueError("this attention does not read another layer call's cache")
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key/value heads evenly")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.eps = float(scale), float(eps)
        self.bias, self.qk_norm, self.sink, self.gate = bias, qk_norm, sink, gate
        self.stretch_coef, self.stretch_every = float(stretch_coef), int(stretch_every)
        self.window = window
        self.out_scale = float(out_scale)
        self.q_dim, self.k_dim, self.v_dim = num_heads * key_dim, num_kv_heads * key_dim, num_kv_heads * value_dim
        self.o_dim = num_heads * value_dim
        self.w_in = self.w_o = self.biases = self.norms = self.w_sink = None

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.key_dim, self.window, value_dim=self.value_dim)

    def weight_specs(self, prefix: str):
        h = self.hidden_size
        specs = [WeightSpec(prefix + "q", (self.q_dim, h), COMPUTE), WeightSpec(prefix + "k", (self.k_dim, h), COMPUTE),
                 WeightSpec(prefix + "v", (self.v_dim, h), COMPUTE), WeightSpec(prefix + "o", (h, self.o_dim), COMPUTE)]
        if self.bias:
            specs += [WeightSpec(prefix + n + ".b", (d,), FLOAT32, init=("normal", 0.3))
                      for n, d in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim))]
        if self.qk_norm:
            specs += [WeightSpec(prefix + "q.norm", (self.key_dim,), FLOAT32, init=("uniform", 0.5, 1.5)),
                      WeightSpec(prefix + "k.norm", (self.key_dim,), FLOAT32, init=("uniform", 0.5, 1.5))]
        if self.sink:
            specs.append(WeightSpec(prefix + "sink", (self.num_heads,), FLOAT32, init=("normal", 1.0)))
        if self.gate:
            specs.append(WeightSpec(prefix + "g", (self.o_dim, h), COMPUTE))
        return specs

    def load(self, prefix: str, weights) -> None:
        rows = [weights[prefix + n] for n in ("q", "k", "v")] + ([weights[prefix + "g"]] if self.gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)
        self.biases = [weights[prefix + n + ".b"] for n in ("q", "k", "v")] if self.bias else [None] * 3
        self.norms = [weights[prefix + "q.norm"], weights[prefix + "k.norm"]] if self.qk_norm else [None, None]
        self.w_sink = weights[prefix + "sink"] if self.sink else None

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        nh, nkv, kd, vd = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        width = self.w_in.shape[0]
        # the row stride is a multiple of 8 values so that the rows can feed the tensor-core kernels
        proj = ctx.workspace.get("qkv", (t, _padded(width)), ctx.dtype)[:, :width]
        ops.linear(h, self.w_in, proj, cluster_slices=True)
        ops.qk_norm_kv_write(proj, ctx.batch.positions, nh, nkv, kd, vd, cache.k, cache.v, cache.slot_mapping,
                             *self.biases, *self.norms, eps=self.eps, stretch_coef=self.stretch_coef,
                             stretch_every=self.stretch_every)
        out = ctx.workspace.get("attn_out", (t, self.o_dim), ctx.dtype)
        # with a gate the attention leaves float32 rows and the gate kernel rounds them; without, it writes `out` itself
        attn = ctx.workspace.get("attn_maps", (t, self.o_dim), torch.float32) if self.gate else out
        ops.paged_attention_maps(proj, nh, nkv, 1, kd, vd, cache.k, cache.v, cache.block_table, ctx.batch, attn,
                                 self.scale, self.window, None, sink=self.w_sink, workspace=ctx.workspace)
        if self.gate:
            off = self.q_dim + self.k_dim + self.v_dim
            ops.sigmoid_gate(attn, proj[:, off:off + self.o_dim], nh, vd, out)
        ops.linear(out, self.w_o, resid, accumulate=True)


class LatentAttention:
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, plain_dim: int, rot_part: int, value_dim: int, rank: int,
                 scale: float, eps: float, rot_dims: int = 0, rot_base: float = 10000.0, window: Optional[int] = None,
                 sink: bool = True, out_scale: float = 1.0, shares_cache: bool = False):
        if shares_cache:
            raise ValueError("this attention does not read another layer call's cache")
        if rot_dims % 2 or rot_dims > rot_part:
            raise ValueError(f"{rot_dims} rotated values must be even and at most the rotated part's size {rot_part}")
        if plain_dim < 1:
            raise ValueError("the queries need a part that is not rotated")
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.plain_dim, self.rot_part, self.value_dim, self.rank = plain_dim, rot_part, value_dim, rank
        self.scale, self.eps = float(scale), float(eps)
        self.rot_dims, self.rot_base = rot_dims, float(rot_base)
        self.window, self.sink = window, sink
        self.out_scale = float(out_scale)
        self.q_dim = num_heads * (plain_dim + rot_part)
        self.key_dim = rank + rot_part          # a cached key row: [latent | rotated part]
        self.w_in = self.w_o = self.w_norm = self.w_sink = self.freq = None
        self.w_uk_t = self.w_uv = None

    def cache_need(self):
        return KVNeed(1, self.key_dim, self.window, value_dim=self.rank)

    def weight_specs(self, prefix: str):
        h, nh = self.hidden_size, self.num_heads
        specs = [WeightSpec(prefix + "q", (self.q_dim, h), COMPUTE),
                 WeightSpec(prefix + "dkv", (self.key_dim, h), COMPUTE),
                 WeightSpec(prefix + "dkv.norm", (self.rank,), FLOAT32, init=("uniform", 0.5, 1.5)),
                 WeightSpec(prefix + "uk", (nh * self.plain_dim, self.rank), COMPUTE),
                 WeightSpec(prefix + "uv", (nh * self.value_dim, self.rank), COMPUTE),
                 WeightSpec(prefix + "g", (nh, h), COMPUTE),
                 WeightSpec(prefix + "o", (h, nh * self.value_dim), COMPUTE)]
        if self.sink:
            specs.append(WeightSpec(prefix + "sink", (nh,), FLOAT32, init=("normal", 1.0)))
        return specs

    def load(self, prefix: str, weights) -> None:
        nh, nd, vd = self.num_heads, self.plain_dim, self.value_dim
        self.w_in = torch.cat([weights[prefix + n] for n in ("q", "dkv", "g")], dim=0).contiguous()
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)
        self.w_norm = weights[prefix + "dkv.norm"]
        self.w_sink = weights[prefix + "sink"] if self.sink else None
        uk, uv = weights[prefix + "uk"], weights[prefix + "uv"]
        # per head: the keys' up-projection transposed (it takes the plain query part into the latent's space) and
        # the values' up-projection as it is, each stacked [heads, outputs, inputs] for the per-head product
        self.w_uk_t = uk.view(nh, nd, self.rank).transpose(1, 2).contiguous()
        self.w_uv = uv.view(nh, vd, self.rank).contiguous()
        self.freq = pair_frequencies(self.rot_dims, self.rot_base).to(self.w_o.device) if self.rot_dims else None

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        nh, nd, rd, vd, rank, kd = self.num_heads, self.plain_dim, self.rot_part, self.value_dim, self.rank, self.key_dim
        qd = nd + rd
        width = self.w_in.shape[0]
        proj = ctx.workspace.get("qkv", (t, _padded(width)), ctx.dtype)[:, :width]
        ops.linear(h, self.w_in, proj, cluster_slices=True)
        q_lat = ctx.workspace.get("latent_q", (t, nh, kd), ctx.dtype)
        ops.latent_kv_write(proj, ctx.batch.positions, nh, nd, rd, rank, self.rot_dims, self.freq, self.w_norm, self.eps,
                            q_lat, cache.k, cache.v, cache.slot_mapping)
        ops.head_linear(proj[:, :nh * qd].view(t, nh, qd)[:, :, :nd], self.w_uk_t, q_lat[:, :, :rank])
        attn = ctx.workspace.get("attn_maps", (t, nh * rank), torch.float32)
        ops.paged_attention_maps(q_lat.view(t, nh * kd), nh, 1, 1, kd, rank, cache.k, cache.v, cache.block_table,
                                 ctx.batch, attn, self.scale, self.window, None, sink=self.w_sink, workspace=ctx.workspace)
        gated = ctx.workspace.get("latent_o", (t, nh * rank), ctx.dtype)
        ops.sigmoid_gate(attn, proj[:, self.q_dim + kd:self.q_dim + kd + nh], nh, rank, gated)
        out = ctx.workspace.get("attn_out", (t, nh * vd), ctx.dtype)
        ops.head_linear(gated.view(t, nh, rank), self.w_uv, out.view(t, nh, vd))
        ops.linear(out, self.w_o, resid, accumulate=True)


register_part("mixer", "sink_attention", SinkAttention)
register_part("mixer", "latent_attention", LatentAttention)
