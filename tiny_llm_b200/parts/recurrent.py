"""Recurrent mixers: a state of fixed size per request instead of keys and values.

Linear attention (below minGRU): a matrix state per head, S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, with no
softmax and no denominator.  `Retention` fixes one decay per head; `GatedLinearAttention` computes a decay per key
channel and token from a low-rank projection of the input.  Both normalise every head's output, multiply it by
silu(Wg h) and project it; the state [heads, key size, value size] is 32-bit in the request's state slot.

minGRU.  A gated recurrence whose gates read the current token only, so all gates of a portion come from one
matrix product and only the element-wise recurrence walks the tokens:
    z_t = sigmoid(Wz h_t + bz)                      how much of the candidate enters
    u_t = Wx h_t + bx;  c_t = u_t + 1/2 (u_t >= 0), sigmoid(u_t) (u_t < 0)      the candidate, always positive
    S_t = (1 - z_t) S_(t-1) + z_t c_t               element by element, S_(-1) = 0
    y_t = Wo (S_t * silu(Wg h_t))
The three input matrices are fused into one at load ([z | u | g] rows); the state is a float32 vector of `width`
values in the request's state slot, carried from step to step; biases, sigmoids and the recurrence are 32-bit."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateNeed
from ..weights import COMPUTE, FLOAT32, WeightSpec
from .feed_forward import scaled_matrix
from .registry import register_part


class MinGRU:
    graph_safe = True   # launches kernels only: a step through this part can be captured in a CUDA graph

    def __init__(self, hidden_size: int, width: int, out_scale: float = 1.0, shares_cache: bool = False):
        if shares_cache:
            raise ValueError("a recurrent mixer's state cannot be read by another layer call")
        self.hidden_size = hidden_size
        self.width = width
        self.out_scale = float(out_scale)
        self.w_in = self.w_o = self.bias_z = self.bias_u = None

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def weight_specs(self, prefix: str):
        w, h = self.width, self.hidden_size
        return [WeightSpec(prefix + "z", (w, h), COMPUTE), WeightSpec(prefix + "z.b", (w,), FLOAT32, init=("normal", 0.5)),
                WeightSpec(prefix + "x", (w, h), COMPUTE), WeightSpec(prefix + "x.b", (w,), FLOAT32, init=("normal", 0.5)),
                WeightSpec(prefix + "g", (w, h), COMPUTE), WeightSpec(prefix + "o", (h, w), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.w_in = torch.cat([weights[prefix + n] for n in ("z", "x", "g")], dim=0).contiguous()
        self.bias_z = weights[prefix + "z.b"]
        self.bias_u = weights[prefix + "x.b"]
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        zug = ctx.workspace.get("gru_in", (t, 3 * self.width), ctx.dtype)
        ops.linear(h, self.w_in, zug, cluster_slices=True)
        y = ctx.workspace.get("gru_out", (t, self.width), ctx.dtype)
        ops.min_gru_scan(zug, self.bias_z, self.bias_u, cache.state, ctx.batch, y, ctx.workspace)
        ops.linear(y, self.w_o, resid, accumulate=True)


register_part("mixer", "min_gru", MinGRU)


class LinearAttention:
    """S_t = diag(a_t) S_(t-1) + (ks k_t) v_t^T;  o_t = S_t^T (qs q_t);  y_t = Wo (norm(o_t) * silu(Wg h_t)), head by head.

    The decay a_t is what the subclasses differ in.  The input matrices are fused into one product at load
    ([q | k | v | g | more] rows); the decays, the recurrence, the state and the norm are 32-bit, the projections are
    the engine's dtype.  `norm_weight`: the per-head norm multiplies by a learned vector of the value size (shared by
    the heads) stored as `<prefix>norm`; without it the head's output is only divided by its root mean square."""
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, eps: float,
                 q_scale: float = 1.0, k_scale: float = 1.0, norm_weight: bool = False, out_scale: float = 1.0,
                 shares_cache: bool = False):
        if shares_cache:
            raise ValueError("a recurrent mixer's state cannot be read by another layer call")
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = hidden_size, num_heads, key_dim, value_dim
        self.eps, self.q_scale, self.k_scale = float(eps), float(q_scale), float(k_scale)
        self.norm_weight = norm_weight
        self.out_scale = float(out_scale)
        self.qk = num_heads * key_dim
        self.vg = num_heads * value_dim
        self.w_in = self.w_o = self.w_norm = None

    def cache_need(self):
        return StateNeed((self.num_heads, self.key_dim, self.value_dim), torch.float32)

    # what a subclass adds
    def extra_rows(self) -> int:
        """Rows the subclass appends to the fused input matrix (behind q, k, v, g)."""
        return 0

    def extra_weight_specs(self, prefix: str):
        return []

    def extra_load(self, prefix: str, weights):
        return []

    def decay_args(self, ctx, proj) -> dict:
        raise NotImplementedError

    def weight_specs(self, prefix: str):
        h = self.hidden_size
        specs = [WeightSpec(prefix + "q", (self.qk, h), COMPUTE), WeightSpec(prefix + "k", (self.qk, h), COMPUTE),
                 WeightSpec(prefix + "v", (self.vg, h), COMPUTE), WeightSpec(prefix + "g", (self.vg, h), COMPUTE),
                 WeightSpec(prefix + "o", (h, self.vg), COMPUTE)]
        if self.norm_weight:
            specs.append(WeightSpec(prefix + "norm", (self.value_dim,), FLOAT32))
        return specs + self.extra_weight_specs(prefix)

    def load(self, prefix: str, weights) -> None:
        rows = [weights[prefix + n] for n in ("q", "k", "v", "g")] + self.extra_load(prefix, weights)
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)
        self.w_norm = weights[prefix + "norm"] if self.norm_weight else None

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        qk, vg = self.qk, self.vg
        width = 2 * qk + 2 * vg + self.extra_rows()
        # the row stride is a multiple of 8 values so that a slice of the rows can feed a tensor-core product
        proj = ctx.workspace.get("lin_attn_in", (t, -(-width // 8) * 8), ctx.dtype)[:, :width]
        ops.linear(h, self.w_in, proj, cluster_slices=True)
        o = ctx.workspace.get("lin_attn_o", (t, vg), torch.float32)
        ops.linear_attention_scan(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vg], self.num_heads,
                                  self.key_dim, self.value_dim, cache.state, ctx.batch, o, self.q_scale, self.k_scale,
                                  workspace=ctx.workspace, **self.decay_args(ctx, proj))
        y = ctx.workspace.get("lin_attn_y", (t, vg), ctx.dtype)
        ops.head_norm_gate(o, self.w_norm, proj[:, 2 * qk + vg:2 * qk + 2 * vg], self.num_heads, self.value_dim,
                           self.eps, y)
        ops.linear(y, self.w_o, resid, accumulate=True)


class Retention(LinearAttention):
    """Linear attention with one fixed decay per head (a_t = decay_h for every key channel and token); keys are
    scaled by key_dim^(-1/2); every head's output is divided by its root mean square, without a weight."""

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay, eps: float, **kw):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, k_scale=key_dim ** -0.5, **kw)
        self.decay = tuple(float(d) for d in decay)
        self.decay_dev = None

    def extra_load(self, prefix, weights):
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=weights[prefix + "o"].device)
        return []

    def decay_args(self, ctx, proj):
        return {"head_decay": self.decay_dev}


class GatedLinearAttention(LinearAttention):
    """Linear attention with a decay per key channel and token: a_t = sigmoid(Wa2 (Wa1 h_t) + b)^(1/tau), a low-rank
    projection (rank = rows of Wa1).  Queries are scaled by key_dim^(-1/2); every head's output is RMS-normed with a
    weight of the value size.  Wa1 rides in the fused input product; the second product leaves 32-bit rows, and the
    bias, the sigmoid and the power are taken in 32-bit inside the recurrence kernel."""

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, tau: float, eps: float,
                 rank: int = 0, **kw):
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, q_scale=key_dim ** -0.5, norm_weight=True, **kw)
        self.tau = float(tau)
        self.rank = rank          # 0: read from the stored tensor's shape
        self.w_a2 = self.b_a2 = None

    def extra_weight_specs(self, prefix):
        r = self.rank if self.rank else None    # None: any number of rows
        return [WeightSpec(prefix + "a1", (r, self.hidden_size), COMPUTE), WeightSpec(prefix + "a2", (self.qk, r), COMPUTE),
                WeightSpec(prefix + "a2.b", (self.qk,), FLOAT32, init=("normal", 1.0))]

    def extra_load(self, prefix, weights):
        a1 = weights[prefix + "a1"]
        self.rank = a1.shape[0]
        a2 = weights[prefix + "a2"]
        if a2.shape[1] != self.rank:
            raise ValueError(f"{prefix}a2 has {a2.shape[1]} columns, {prefix}a1 {self.rank} rows")
        pad = -(-self.rank // 8) * 8     # K of the second product as a multiple of 8 (zero columns add nothing)
        self.w_a2 = torch.zeros(self.qk, pad, dtype=a2.dtype, device=a2.device)
        self.w_a2[:, :self.rank] = a2
        self.b_a2 = weights[prefix + "a2.b"]
        self._pad = pad - self.rank
        return [a1] + ([torch.zeros(self._pad, self.hidden_size, dtype=a1.dtype, device=a1.device)] if self._pad else [])

    def extra_rows(self):
        return self.w_a2.shape[1] if self.w_a2 is not None else self.rank

    def decay_args(self, ctx, proj):
        t = proj.shape[0]
        off = 2 * self.qk + 2 * self.vg
        z = ctx.workspace.get("lin_attn_gate", (t, self.qk), torch.float32)
        ops.linear(proj[:, off:off + self.w_a2.shape[1]], self.w_a2, z)
        return {"gate": z, "gate_bias": self.b_a2, "inv_tau": 1.0 / self.tau}


class GatedDeltaRule:
    """The gated delta rule: per head a matrix state that is decayed, corrected towards the current value along the
    current key, and read out with the query,
        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's write)
    with beta = sigmoid(Wb h), g = exp(-exp(A_log) softplus(Wa h + dt_bias)), one of each per head and token.  q and k
    have `num_kv_heads` heads (head h reads head h // (heads / kv_heads)), v has `num_heads`; each of q, k, v passes a
    short causal convolution over time (a filter of `taps` values per channel, stored `<tensor>.conv`, its last column
    at the current token, no bias) and SiLU; q and k are made unit vectors per head, x / sqrt(sum(x^2) + unit_eps), q
    also times key_dim^(-1/2).  Every head's o is divided by its root mean square, multiplied by a weight of the value
    size and by silu(Wg h), and projected.

    All input matrices are one product ([q | k | v | g | b | a] rows).  Per request the mixer keeps two things in the
    state slot, both 32-bit: S transposed ([heads, value, key]) and the last taps - 1 inputs of every convolution
    channel.  Decays, step sizes, unit norms, the recurrence and the per-head norm are 32-bit.

    `decay="channel"`: one decay per head AND key channel, S <- diag(g) S with g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 h)
    + dt_bias)) laid out heads x key size (a low-rank projection stored as `a1`, `a2`; `dt_bias` has heads x key size
    values; there is no `a`).  `gate_act="sigmoid"` multiplies the normed output by sigmoid instead of silu;
    `gate_low_rank=True` takes the gate's input from a low-rank projection Wg2 (Wg1 h) stored as `g1`, `g2` instead
    of `g`.  The ranks are read from the stored tensors."""
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, taps: int,
                 eps: float, unit_eps: float = 1e-6, decay: str = "head", gate_act: str = "silu",
                 gate_low_rank: bool = False, out_scale: float = 1.0, shares_cache: bool = False):
        if decay not in ("head", "channel"):
            raise ValueError(f"unknown decay kind {decay!r} (known: head, channel)")
        if gate_act not in ("silu", "sigmoid"):
            raise ValueError(f"unknown gate activation {gate_act!r} (known: silu, sigmoid)")
        self.decay, self.gate_act, self.gate_low_rank = decay, gate_act, gate_low_rank
        if shares_cache:
            raise ValueError("a recurrent mixer's state cannot be read by another layer call")
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} query/key heads evenly")
        if taps < 1:
            raise ValueError("a convolution has at least one tap")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim, self.taps = key_dim, value_dim, taps
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.out_scale = float(out_scale)
        self.qk = num_kv_heads * key_dim
        self.vg = num_heads * value_dim
        self.channels = 2 * self.qk + self.vg
        self.w_in = self.w_o = self.w_taps = self.w_norm = self.a_log = self.dt_bias = None
        self.w_a2 = self.w_g2 = None
        self.gate_cols = self.decay_cols = 0      # columns of the fused projection behind the channels / behind b

    def cache_need(self):
        return (StateNeed((self.num_heads, self.value_dim, self.key_dim), torch.float32),
                StateNeed((max(self.taps - 1, 1), self.channels), torch.float32))

    def weight_specs(self, prefix: str):
        h, nh = self.hidden_size, self.num_heads
        taps = ("normal", 0.5)
        specs = [WeightSpec(prefix + "q", (self.qk, h), COMPUTE), WeightSpec(prefix + "q.conv", (self.qk, self.taps), FLOAT32, init=taps),
                 WeightSpec(prefix + "k", (self.qk, h), COMPUTE), WeightSpec(prefix + "k.conv", (self.qk, self.taps), FLOAT32, init=taps),
                 WeightSpec(prefix + "v", (self.vg, h), COMPUTE), WeightSpec(prefix + "v.conv", (self.vg, self.taps), FLOAT32, init=taps),
                 WeightSpec(prefix + "b", (nh, h), COMPUTE),
                 WeightSpec(prefix + "A_log", (nh,), FLOAT32, init=("uniform", -3.0, 0.5)),
                 WeightSpec(prefix + "norm", (self.value_dim,), FLOAT32, init=("uniform", 0.5, 1.5)),
                 WeightSpec(prefix + "o", (h, self.vg), COMPUTE)]
        if self.decay == "channel":
            specs += [WeightSpec(prefix + "a1", (None, h), COMPUTE, free_dim=12),
                      WeightSpec(prefix + "a2", (nh * self.key_dim, None), COMPUTE, free_dim=12, init=("normal", 0.5)),
                      WeightSpec(prefix + "dt_bias", (nh * self.key_dim,), FLOAT32, init=("normal", 1.0))]
        else:
            specs += [WeightSpec(prefix + "a", (nh, h), COMPUTE), WeightSpec(prefix + "dt_bias", (nh,), FLOAT32, init=("normal", 1.0))]
        if self.gate_low_rank:
            specs += [WeightSpec(prefix + "g1", (None, h), COMPUTE, free_dim=12),
                      WeightSpec(prefix + "g2", (self.vg, None), COMPUTE, free_dim=12, init=("normal", 0.5))]
        else:
            specs.append(WeightSpec(prefix + "g", (self.vg, h), COMPUTE))
        return specs

    @staticmethod
    def _low_rank(first: torch.Tensor, second: torch.Tensor, names: str):
        """The two matrices of a low-rank projection with the rank padded to a multiple of 8 (zero rows of the first
        and zero columns of the second add nothing), so that the second product can run on the tensor cores."""
        rank = first.shape[0]
        if second.shape[1] != rank:
            raise ValueError(f"{names}: {second.shape[1]} columns against {rank} rows")
        pad = -(-rank // 8) * 8
        a = torch.zeros(pad, first.shape[1], dtype=first.dtype, device=first.device)
        a[:rank] = first
        b = torch.zeros(second.shape[0], pad, dtype=second.dtype, device=second.device)
        b[:, :rank] = second
        return a, b

    def load(self, prefix: str, weights) -> None:
        rows = [weights[prefix + n] for n in ("q", "k", "v")]
        if self.gate_low_rank:
            g1, self.w_g2 = self._low_rank(weights[prefix + "g1"], weights[prefix + "g2"], prefix + "g1/g2")
            rows.append(g1)
            self.gate_cols = g1.shape[0]
        else:
            rows.append(weights[prefix + "g"])
            self.gate_cols = self.vg
        rows.append(weights[prefix + "b"])
        if self.decay == "channel":
            a1, self.w_a2 = self._low_rank(weights[prefix + "a1"], weights[prefix + "a2"], prefix + "a1/a2")
            rows.append(a1)
            self.decay_cols = a1.shape[0]
        else:
            rows.append(weights[prefix + "a"])
            self.decay_cols = self.num_heads
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_taps = torch.cat([weights[prefix + n + ".conv"] for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)
        self.w_norm, self.a_log, self.dt_bias = weights[prefix + "norm"], weights[prefix + "A_log"], weights[prefix + "dt_bias"]

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        nh, nkv, kd, vd, ws = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim, ctx.workspace
        state, kept = cache
        c, vg = self.channels, self.vg
        b_col = c + self.gate_cols
        a_col = b_col + nh
        width = a_col + self.decay_cols
        proj = ws.get("lin_attn_in", (t, -(-width // 8) * 8), ctx.dtype)[:, :width]
        ops.linear(h, self.w_in, proj, cluster_slices=True)
        q = ws.get("delta_q", (t, self.qk), torch.float32)
        k = ws.get("delta_k", (t, self.qk), torch.float32)
        v = ws.get("delta_v", (t, vg), torch.float32)
        gb = ws.get("delta_gb", (t, nh, 2), torch.float32)
        more, mode = {}, "delta"
        if self.decay == "channel":   # the second product of the decays' projection leaves 32-bit rows
            mode = "channel_decay"
            decay_in = ws.get("delta_decay_in", (t, nh * kd), torch.float32)
            ops.linear(proj[:, a_col:a_col + self.decay_cols], self.w_a2, decay_in)
            more = {"decay_in": decay_in, "gk": ws.get("delta_gk", (t, nh * kd), torch.float32)}
        ops.delta_prepare(proj, self.w_taps, kept.state, ctx.batch, nh, nkv, kd, vd, b_col, a_col, self.a_log,
                          self.dt_bias, kd ** -0.5, self.unit_eps, q, k, v, gb, mode=mode, **more)
        ops.conv_state_update(proj, kept.state, ctx.batch, self.taps, c)
        o = ws.get("lin_attn_o", (t, vg), torch.float32)
        ops.delta_rule_scan(q, k, v, gb, state.state, ctx.batch, nh, nkv, kd, vd, o, mode=mode, gk=more.get("gk"))
        y = ws.get("lin_attn_y", (t, vg), ctx.dtype)
        gate = proj[:, c:c + vg]
        if self.gate_low_rank:
            gate = ws.get("delta_gate", (t, vg), ctx.dtype)
            ops.linear(proj[:, c:c + self.gate_cols], self.w_g2, gate)
        ops.head_norm_gate(o, self.w_norm, gate, nh, vd, self.eps, y, act=self.gate_act)
        ops.linear(y, self.w_o, resid, accumulate=True)


class Mamba2:
    """The state-space mixer in its scalar-decay form: per head a matrix state S [state size, value size],
        S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x
    with the step size dt = softplus(dt_in + dt_bias) per head and token.  One product gives [z | x | B | C | dt_in]
    (z and x of heads * value_dim values, B and C of groups * state_dim, head h reading group h // (heads / groups));
    x, B and C pass a short causal convolution per channel with a bias (`conv` [channels, taps], last column at the
    current token, `conv.b`) and SiLU.  The joined heads are multiplied by silu(z) FIRST and then divided by the root
    mean square of each of `norm_parts` equal parts of the row, times a weight of the row's size, then projected.
    Per request the mixer keeps S transposed ([heads, value, state], 32-bit) and the convolutions' last taps - 1
    inputs.  Step sizes, decays, the recurrence, the skip and the norm are 32-bit.  The recurrence is the delta rule's
    kernel without its correction term (keys = B, queries = C, values = x, step size = dt)."""
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, value_dim: int, state_dim: int, groups: int, taps: int,
                 norm_parts: int, eps: float, out_scale: float = 1.0, shares_cache: bool = False):
        if shares_cache:
            raise ValueError("a recurrent mixer's state cannot be read by another layer call")
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads cannot share {groups} groups evenly")
        if (num_heads * value_dim) % norm_parts:
            raise ValueError(f"a row of {num_heads * value_dim} values cannot be normed in {norm_parts} equal parts")
        if taps < 1:
            raise ValueError("a convolution has at least one tap")
        self.hidden_size, self.num_heads, self.value_dim, self.state_dim = hidden_size, num_heads, value_dim, state_dim
        self.groups, self.taps, self.norm_parts, self.eps = groups, taps, norm_parts, float(eps)
        self.out_scale = float(out_scale)
        self.inner = num_heads * value_dim
        self.bc = groups * state_dim
        self.channels = self.inner + 2 * self.bc
        self.w_in = self.w_o = self.w_taps = self.b_taps = self.w_norm = self.a_log = self.dt_bias = self.skip = None

    def cache_need(self):
        return (StateNeed((self.num_heads, self.value_dim, self.state_dim), torch.float32),
                StateNeed((max(self.taps - 1, 1), self.channels), torch.float32))

    def weight_specs(self, prefix: str):
        h, nh = self.hidden_size, self.num_heads
        return [WeightSpec(prefix + "in", (self.inner + self.channels + nh, h), COMPUTE),
                WeightSpec(prefix + "conv", (self.channels, self.taps), FLOAT32, init=("normal", 0.5)),
                WeightSpec(prefix + "conv.b", (self.channels,), FLOAT32, init=("normal", 0.2)),
                WeightSpec(prefix + "dt_bias", (nh,), FLOAT32, init=("normal", 1.0)),
                WeightSpec(prefix + "A_log", (nh,), FLOAT32, init=("uniform", -3.0, 0.5)),
                WeightSpec(prefix + "D", (nh,), FLOAT32, init=("normal", 1.0)),
                WeightSpec(prefix + "norm", (self.inner,), FLOAT32, init=("uniform", 0.5, 1.5)),
                WeightSpec(prefix + "o", (h, self.inner), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.w_in = weights[prefix + "in"]
        self.w_taps, self.b_taps = weights[prefix + "conv"], weights[prefix + "conv.b"]
        self.dt_bias, self.a_log, self.skip = weights[prefix + "dt_bias"], weights[prefix + "A_log"], weights[prefix + "D"]
        self.w_norm = weights[prefix + "norm"]
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        nh, vd, n, ws = self.num_heads, self.value_dim, self.state_dim, ctx.workspace
        state, kept = cache
        inner, c = self.inner, self.channels
        width = inner + c + nh
        proj = ws.get("lin_attn_in", (t, -(-width // 8) * 8), ctx.dtype)[:, :width]
        ops.linear(h, self.w_in, proj, cluster_slices=True)
        conv_in = proj[:, inner:]                 # [x | B | C | dt_in]
        q = ws.get("delta_q", (t, self.bc), torch.float32)    # C
        k = ws.get("delta_k", (t, self.bc), torch.float32)    # B
        v = ws.get("delta_v", (t, inner), torch.float32)      # x
        gb = ws.get("delta_gb", (t, nh, 2), torch.float32)    # (decay, dt)
        ops.delta_prepare(conv_in, self.w_taps, kept.state, ctx.batch, nh, self.groups, n, vd, c, c, self.a_log,
                          self.dt_bias, 1.0, 0.0, q, k, v, gb, mode="state_space", conv_bias=self.b_taps)
        ops.conv_state_update(conv_in, kept.state, ctx.batch, self.taps, c)
        o = ws.get("lin_attn_o", (t, inner), torch.float32)
        ops.delta_rule_scan(q, k, v, gb, state.state, ctx.batch, nh, self.groups, n, vd, o, mode="state_space")
        y = ws.get("lin_attn_y", (t, inner), ctx.dtype)
        ops.gated_group_norm(o, proj[:, :inner], self.w_norm, self.norm_parts, vd, self.eps, y, skip_x=v, skip=self.skip)
        ops.linear(y, self.w_o, resid, accumulate=True)


register_part("mixer", "mamba2", Mamba2)


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
register_part("mixer", "retention", Retention)
register_part("mixer", "gated_linear_attention", GatedLinearAttention)
