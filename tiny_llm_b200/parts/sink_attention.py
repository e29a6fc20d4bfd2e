"""Softmax attention with a sink and an output gate, in two forms.

Both share the softmax: beside the visible keys' terms its denominator holds exp(sink_h), a learned score per head
that stands for no key and has no value, so a head may give weight to nothing.  Both multiply the heads' outputs by
sigmoid(Wg h) of the mixer's own input before the output projection.  Scores, the softmax, norms, angles and the
gate's sigmoid are 32-bit; the attention kernel leaves float32 rows and the gate kernel rounds them once.

`SinkAttention`: grouped-query heads with optional biases on q, k, v, optional norms of every query and key head
(x / sqrt(mean(x^2) + eps) * w, one weight vector of the key size for all heads), no rotation, and optionally a query
that grows with the logarithm of its position, q <- q (1 + coef ln(floor((p + 1) / every) + 1)).  Key size and value
size may differ.  The gate has one value per output value, or one per head (`gate="head"`).  Further options:
`rot_dims` > 0 turns the first rot_dims values of every query and key head behind the norm, value i with i + rot_dims / 2
(`rot_layout="halves"`) or 2i with 2i + 1 ("pairs"), by p * f_i with the frequencies of `stretched_frequencies`;
`head_temp` multiplies head h's scores by a learned number `temp`[h]; `talk` mixes the heads' scores before the softmax,
z_h = sum_g talk[h, g] s_g with a learned heads x heads matrix.  With either of the last two the scores of all heads
meet in one kernel (`ops.attention_talk`), which takes scale, temperatures and mixing as ONE matrix
M[h, g] = talk[h, g] * temp[g] * scale (made in 32-bit at load).

`LatentAttention`: keys and values of all heads are projections of ONE small latent vector per token,
    c = norm(first `rank` rows of Wdkv h),   k_h = [Wuk_h c | rot(last rows of Wdkv h)],   v_h = Wuv_h c,
and the queries are [plain | rotated] per head.  Only c and the rotated key part are cached.  The scores are taken
against the cache as it is: with q'_h = Wuk_h^T q_plain_h the score q_plain_h . (Wuk_h c) equals q'_h . c, so every
head attends with the query [q'_h | q_rot_h] over one shared key row [c | k_rot] and one shared value row c, and the
head's value projection is applied to the weighted sum of latents afterwards: o_h = Wuv_h (sum_j p_j c_j).  The rotated
parts turn in pairs (2i, 2i + 1) by p * base^(-2i / rot_dims).  A key is visible while 0 <= i - j < window.  The gate
has one value per head (`gate=False`: none).  Built with `shares_cache=True` (a run-order entry that reads another
entry's cache) the mixer has no Wdkv and no latent norm: it attends over the latents and rotated key parts that the
other layer cached, with its own Wuk, Wuv, queries and sink."""
from __future__ import annotations

import math
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


def stretched_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
    """The rotation frequencies f_i = base^(-2i / dims), i < dims / 2, and the factor that cos and sin are multiplied
    by.  `scaling` = {"factor", "original", "fast", "slow"} stretches a model's positions past the `original` length
    it was trained on: a pair that turns more than `fast` times over that length keeps its frequency, one that turns
    fewer than `slow` times is slowed by `factor`, and the pairs between blend the two linearly in the pair's index,
        d(t) = dims ln(original / (2 pi t)) / (2 ln base),  lo = max(floor(d(fast)), 0),  hi = min(ceil(d(slow)), dims - 1),
        r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),   f_i <- f_i / factor * r_i + f_i (1 - r_i),
    and the magnitude grows to 0.1 ln(factor) + 1.  Computed in 64-bit, kept in 32-bit."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    mag = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def pair_of(turns: float) -> float:
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
        lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    return f.to(torch.float32).contiguous(), mag


def _padded(n: int) -> int:
    return -(-n // 8) * 8


class SinkAttention:
    graph_safe = True   # launches kernels only

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 eps: float, bias: bool = True, qk_norm: bool = True, sink: bool = True, gate: bool = True,
                 stretch_coef: float = 0.0, stretch_every: int = 0, window: Optional[int] = None,
                 rot_dims: int = 0, rot_base: float = 10000.0, rot_scaling: Optional[dict] = None,
                 rot_layout: str = "halves", head_temp: bool = False, talk: bool = False,
                 out_scale: float = 1.0, shares_cache: bool = False):
        if shares_cache:
            raise ValueError("this attention does not read another layer call's cache")
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key/value heads evenly")
        if rot_dims % 2 or rot_dims > key_dim or rot_layout not in ("halves", "pairs"):
            raise ValueError(f"{rot_dims} rotated values must be even and at most the key size {key_dim}; layouts: halves, pairs")
        if gate not in (True, False, "head"):
            raise ValueError(f"unknown gate kind {gate!r} (True: one per value, \"head\": one per head, False: none)")
        self.rot_dims, self.rot_base, self.rot_scaling, self.rot_layout = rot_dims, float(rot_base), rot_scaling, rot_layout
        self.head_temp, self.talk = head_temp, talk
        self.freq, self.rot_mag, self.mix, self.mix_log2 = None, 1.0, None, None
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.eps = float(scale), float(eps)
        self.bias, self.qk_norm, self.sink, self.gate = bias, qk_norm, sink, gate
        self.stretch_coef, self.stretch_every = float(stretch_coef), int(stretch_every)
        self.window = window
        self.out_scale = float(out_scale)
        self.q_dim, self.k_dim, self.v_dim = num_heads * key_dim, num_kv_heads * key_dim, num_kv_heads * value_dim
        self.o_dim = num_heads * value_dim
        self.g_dim = 0 if not gate else (num_heads if gate == "head" else self.o_dim)
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
            specs.append(WeightSpec(prefix + "g", (self.g_dim, h), COMPUTE))
        if self.head_temp:
            specs.append(WeightSpec(prefix + "temp", (self.num_heads,), FLOAT32, init=("uniform", 0.6, 1.6)))
        if self.talk:
            specs.append(WeightSpec(prefix + "talk", (self.num_heads, self.num_heads), FLOAT32, init=("normal", 0.4)))
        return specs

    def load(self, prefix: str, weights) -> None:
        rows = [weights[prefix + n] for n in ("q", "k", "v")] + ([weights[prefix + "g"]] if self.gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        if self.rot_dims:
            self.freq, self.rot_mag = stretched_frequencies(self.rot_dims, self.rot_base, self.rot_scaling)
            self.freq = self.freq.to(self.w_in.device)
        if self.head_temp or self.talk:
            nh = self.num_heads
            mix = weights[prefix + "talk"].to(torch.float32) if self.talk else torch.eye(nh, device=self.w_in.device)
            if self.head_temp:
                mix = mix * weights[prefix + "temp"].to(torch.float32)[None, :]
            self.mix = (mix * self.scale).contiguous()
            self.mix_log2 = (self.mix.double() * math.log2(math.e)).to(torch.float32).contiguous()   # powers of two in the tensor-core kernel
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
                             stretch_every=self.stretch_every, freq=self.freq, rot_pairs=self.rot_layout == "pairs",
                             rot_mag=self.rot_mag)
        out = ctx.workspace.get("attn_out", (t, self.o_dim), ctx.dtype)
        off = self.q_dim + self.k_dim + self.v_dim
        if self.mix is not None:    # all heads' scores meet: one kernel, which also applies a gate per head
            per_head = self.gate == "head"
            attn = ctx.workspace.get("attn_maps", (t, self.o_dim), torch.float32) if self.gate and not per_head else out
            ops.attention_talk(proj, nh, nkv, kd, vd, cache.k, cache.v, cache.block_table, ctx.batch, self.mix, attn,
                               window=self.window, sink=self.w_sink, gate=proj[:, off:off + nh] if per_head else None,
                               mix_log2=self.mix_log2, workspace=ctx.workspace)
            if self.gate and not per_head:
                ops.sigmoid_gate(attn, proj[:, off:off + self.o_dim], nh, vd, out)
            ops.linear(out, self.w_o, resid, accumulate=True)
            return
        # with a gate the attention leaves float32 rows and the gate kernel rounds them; without, it writes `out` itself
        attn = ctx.workspace.get("attn_maps", (t, self.o_dim), torch.float32) if self.gate else out
        ops.paged_attention_maps(proj, nh, nkv, 1, kd, vd, cache.k, cache.v, cache.block_table, ctx.batch, attn,
                                 self.scale, self.window, None, sink=self.w_sink, workspace=ctx.workspace)
        if self.gate:
            ops.sigmoid_gate(attn, proj[:, off:off + self.g_dim], nh, vd, out)
        ops.linear(out, self.w_o, resid, accumulate=True)


class LatentAttention:
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, plain_dim: int, rot_part: int, value_dim: int, rank: int,
                 scale: float, eps: float, rot_dims: int = 0, rot_base: float = 10000.0, window: Optional[int] = None,
                 sink: bool = True, gate: bool = True, rot_scaling: Optional[dict] = None, out_scale: float = 1.0,
                 shares_cache: bool = False):
        self.shares_cache, self.gate, self.rot_scaling, self.rot_mag = shares_cache, gate, rot_scaling, 1.0
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
                 WeightSpec(prefix + "uk", (nh * self.plain_dim, self.rank), COMPUTE),
                 WeightSpec(prefix + "uv", (nh * self.value_dim, self.rank), COMPUTE),
                 WeightSpec(prefix + "o", (h, nh * self.value_dim), COMPUTE)]
        if not self.shares_cache:
            specs += [WeightSpec(prefix + "dkv", (self.key_dim, h), COMPUTE),
                      WeightSpec(prefix + "dkv.norm", (self.rank,), FLOAT32, init=("uniform", 0.5, 1.5))]
        if self.gate:
            specs.append(WeightSpec(prefix + "g", (nh, h), COMPUTE))
        if self.sink:
            specs.append(WeightSpec(prefix + "sink", (nh,), FLOAT32, init=("normal", 1.0)))
        return specs

    def load(self, prefix: str, weights) -> None:
        nh, nd, vd = self.num_heads, self.plain_dim, self.value_dim
        rows = ["q"] + ([] if self.shares_cache else ["dkv"]) + (["g"] if self.gate else [])
        self.w_in = torch.cat([weights[prefix + n] for n in rows], dim=0).contiguous()
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)
        self.w_norm = None if self.shares_cache else weights[prefix + "dkv.norm"]
        self.w_sink = weights[prefix + "sink"] if self.sink else None
        uk, uv = weights[prefix + "uk"], weights[prefix + "uv"]
        # per head: the keys' up-projection transposed (it takes the plain query part into the latent's space) and
        # the values' up-projection as it is, each stacked [heads, outputs, inputs] for the per-head product
        self.w_uk_t = uk.view(nh, nd, self.rank).transpose(1, 2).contiguous()
        self.w_uv = uv.view(nh, vd, self.rank).contiguous()
        self.freq = None
        if self.rot_dims:
            self.freq, self.rot_mag = stretched_frequencies(self.rot_dims, self.rot_base, self.rot_scaling)
            self.freq = self.freq.to(self.w_o.device)

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        nh, nd, rd, vd, rank, kd = self.num_heads, self.plain_dim, self.rot_part, self.value_dim, self.rank, self.key_dim
        qd = nd + rd
        width = self.w_in.shape[0]
        proj = ctx.workspace.get("qkv", (t, _padded(width)), ctx.dtype)[:, :width]
        ops.linear(h, self.w_in, proj, cluster_slices=True)
        q_lat = ctx.workspace.get("latent_q", (t, nh, kd), ctx.dtype)
        if self.shares_cache:   # the other layer's step has written the token's rows already; only the queries turn
            ops.latent_kv_write(proj, ctx.batch.positions, nh, nd, rd, rank, self.rot_dims, self.freq, None, self.eps,
                                q_lat, None, None, None, rot_mag=self.rot_mag)
        else:
            ops.latent_kv_write(proj, ctx.batch.positions, nh, nd, rd, rank, self.rot_dims, self.freq, self.w_norm, self.eps,
                                q_lat, cache.k, cache.v, cache.slot_mapping, rot_mag=self.rot_mag)
        ops.head_linear(proj[:, :nh * qd].view(t, nh, qd)[:, :, :nd], self.w_uk_t, q_lat[:, :, :rank])
        attn = ctx.workspace.get("attn_maps", (t, nh * rank), torch.float32)
        ops.paged_attention_maps(q_lat.view(t, nh * kd), nh, 1, 1, kd, rank, cache.k, cache.v, cache.block_table,
                                 ctx.batch, attn, self.scale, self.window, None, sink=self.w_sink, workspace=ctx.workspace)
        gated = ctx.workspace.get("latent_o", (t, nh * rank), ctx.dtype)
        if self.gate:
            g0 = self.q_dim + (0 if self.shares_cache else kd)
            ops.sigmoid_gate(attn, proj[:, g0:g0 + nh], nh, rank, gated)
        else:
            ops.unary(attn, gated)
        out = ctx.workspace.get("attn_out", (t, nh * vd), ctx.dtype)
        ops.head_linear(gated.view(t, nh, rank), self.w_uv, out.view(t, nh, vd))
        ops.linear(out, self.w_o, resid, accumulate=True)


register_part("mixer", "sink_attention", SinkAttention)
register_part("mixer", "latent_attention", LatentAttention)
