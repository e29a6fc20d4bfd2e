"""A plain, slow implementation of the Fiponex decoder, one function per mechanism, written from the design's
equations and sharing no code with the package.  Everything is torch on the CPU in the dtype of the weights it is
handed (float64 for an oracle); recurrences are walked token by token.

The design.  x = embed[token] * s.  A layer norms both sides of each branch:
    x += n1b(mixer(n1(x)));  x += n2b(ff(n2(x)))          n(y) = y / sqrt(mean(y^2) + eps) * (1 + w)
(no second line when the layer has no feed-forward).  Mixers:
  attention         grouped heads with biased q/k/v, q and k normed per head (plain weight), no rotation; the query is
                    stretched by 1 + coef * ln(floor((p + 1) / every) + 1); causal softmax whose denominator also holds
                    exp(sink_h); the joined heads times sigmoid(Wg h); Wo.
  latent_attention  keys and values are projections of one small latent per token, c = norm(first rows of Wdkv h), plus
                    one rotated key part shared by the heads (the last rows of Wdkv h); queries are [plain | rotated]
                    per head; neighbours (2i, 2i + 1) are rotated by p * base^(-2i / dims); a key is seen while
                    0 <= i - j < size; the same sink; head h times sigmoid(Wg h)_h; Wo.
  delta             q, k, v through a short causal convolution per channel and silu; q, k made unit vectors per head
                    (q also / sqrt(dim)); per head S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with
                    beta = sigmoid(Wb h), g = exp(-exp(A_log) softplus(Wa h + dt_bias)); o / rms(o) * w_norm * silu(Wg h); Wo.
Feed-forwards: Wd (relu(Wg h) * (Wu h)), or experts Wd (silu(Wg h) * (Wu h)) chosen by the largest softmax(router)
scores and weighted by those scores as they are."""
from __future__ import annotations

import json
import math
import os

import torch


def no_quant(x):
    return x


def bf16_quant(x):
    """Rounds to bfloat16 and back: what the engine's bfloat16 path does to an activation it stores."""
    return x.to(torch.bfloat16).to(x.dtype)


def load_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def load_weights(model_dir):
    """Reads model.safetensors with this file's own reader: 8 bytes of length, a JSON header, raw little-endian data."""
    import numpy as np
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        n = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = bytes(data[lo:hi])
        if info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        elif info["dtype"] == "BF16":
            t = (torch.from_numpy(np.frombuffer(raw, dtype="<u2").astype(np.int32).copy()) << 16).view(torch.float32)
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(info["dtype"])
        out[name] = t.reshape(info["shape"])
    return out


# ---------------------------------------------------------------------------------------------- small pieces

def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layer norm of the design: the stored weight lies around zero."""
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def query_stretch(pos, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    return 1.0 + coef * torch.log(torch.floor((pos.to(torch.float64) + 1.0) / every) + 1.0)


def rotate_pairs(x, pos, dims, base, angles32=False):
    """x [T, rows, D]: values (2i, 2i + 1), i < dims / 2, of every row turn by pos * base^(-2i / dims).  `angles32`:
    the angle is the 32-bit product of the position and the 32-bit frequency, as the design computes it (at position
    30,000 that differs from the exact angle by a thousandth of a radian)."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    a = pos.to(torch.float64)[:, None, None] * f[None, None, :]
    if angles32:
        a = (pos.to(torch.float32)[:, None, None] * f.to(torch.float32)[None, None, :]).to(torch.float64)
    c, s = torch.cos(a).to(x.dtype), torch.sin(a).to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def sink_softmax_attention(q, k, v, pos_q, pos_k, scale, sink, window=None):
    """q [Tq, heads, D], k [Tk, kv, D], v [Tk, kv, Dv]; head h reads key/value head h // (heads / kv).  A key at
    position j is seen by a query at position i iff j <= i (and i - j < window).  The softmax's denominator holds
    exp(sink_h) beside the seen keys' terms; the sink has no value.  Returns [Tq, heads, Dv]."""
    tq, heads, _ = q.shape
    kv = k.shape[1]
    group = heads // kv
    out = torch.zeros(tq, heads, v.shape[-1], dtype=q.dtype)
    d = pos_q[:, None] - pos_k[None, :]
    seen = d >= 0
    if window is not None:
        seen = seen & (d < window)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // group].T) * scale
        s = torch.where(seen, s, torch.full_like(s, -float("inf")))
        m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[h].to(q.dtype).reshape(1, 1))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True) + torch.exp(sink[h].to(q.dtype) - m)
        out[:, h] = (e / den) @ v[:, h // group]
    return out


def short_conv(x, taps, before=None):
    """x [T, C]; taps [C, n]; y_t = sum_j taps[:, j] * x_(t - (n - 1) + j) (the last column meets the current token;
    zeros, or `before` [n - 1, C], stand ahead of the first token).  Returns y and the last n - 1 inputs."""
    n = taps.shape[1]
    pad = torch.zeros(n - 1, x.shape[1], dtype=x.dtype) if before is None else before.to(x.dtype)
    full = torch.cat([pad, x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + full[j: j + x.shape[0]] * taps[:, j][None, :]
    return y, full[full.shape[0] - (n - 1):]


def delta_rule(q, k, v, beta, g, s0=None):
    """Per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  q, k [T, heads, D], v [T, heads, Dv],
    beta, g [T, heads]; s0 [heads, D, Dv] or None.  Returns o [T, heads, Dv] and the last state."""
    t, heads, dim = q.shape
    vdim = v.shape[-1]
    s = torch.zeros(heads, dim, vdim, dtype=q.dtype) if s0 is None else s0.clone().to(q.dtype)
    out = torch.zeros(t, heads, vdim, dtype=q.dtype)
    for i in range(t):
        for h in range(heads):
            s[h] = g[i, h] * s[h]
            u = beta[i, h] * (v[i, h] - s[h].T @ k[i, h])
            s[h] = s[h] + torch.outer(k[i, h], u)
            out[i, h] = s[h].T @ q[i, h]
    return out, s


def route_softmax(z, top):
    """Scores softmax(z) over all experts; the `top` largest are chosen (ties: the lower index) and keep their scores."""
    s = torch.softmax(z, dim=-1)
    order = torch.argsort(-s, dim=-1, stable=True)[:, :top]
    return order, torch.gather(s, 1, order)


# ---------------------------------------------------------------------------------------------- mixers

def attention_mixer(h, w, p, m, eps, pos, quant=no_quant):
    t = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = quant(h @ w(p + "q").T + w(p + "q.b")).view(t, heads, dim)
    k = quant(h @ w(p + "k").T + w(p + "k.b")).view(t, kv, dim)
    v = quant(h @ w(p + "v").T + w(p + "v.b")).view(t, kv, vdim)
    q = norm_plain(q, w(p + "q.norm"), eps)
    k = quant(norm_plain(k, w(p + "k.norm"), eps))
    qt = m.get("q_temp")
    if qt:
        q = q * query_stretch(pos, qt["coef"], qt["every"]).to(q.dtype)[:, None, None]
    q = quant(q)
    o = sink_softmax_attention(q, k, v, pos, pos, m["scale"], w(p + "sink"))
    gate = torch.sigmoid(quant(h @ w(p + "g").T))
    return quant(o.reshape(t, heads * vdim) * gate) @ w(p + "o").T


def latent_attention_mixer(h, w, p, m, eps, pos, quant=no_quant):
    t = h.shape[0]
    heads, dim, rd, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    q = quant(h @ w(p + "q").T).view(t, heads, dim + rd)
    dkv = quant(h @ w(p + "dkv").T)
    c = quant(norm_plain(dkv[:, :rank], w(p + "dkv.norm"), eps))
    k_rot = dkv[:, rank:].view(t, 1, rd)
    if rot:
        k_rot = rotate_pairs(k_rot, pos, rot["dims"], rot["base"])
        q = torch.cat([q[..., :dim], rotate_pairs(q[..., dim:], pos, rot["dims"], rot["base"])], dim=-1)
    k_rot = quant(k_rot)
    q = quant(q)
    k_plain = (c @ w(p + "uk").T).view(t, heads, dim)
    v = (c @ w(p + "uv").T).view(t, heads, vdim)
    k = torch.cat([k_plain, k_rot.expand(t, heads, rd)], dim=-1)
    window = (m.get("mask") or {}).get("size")
    o = sink_softmax_attention(q, k, v, pos, pos, m["scale"], w(p + "sink"), window)
    gate = torch.sigmoid(quant(h @ w(p + "g").T))
    return quant((o * gate[:, :, None]).reshape(t, heads * vdim)) @ w(p + "o").T


def delta_mixer(h, w, p, m, eps, quant=no_quant):
    t = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    group = heads // kv
    q, _ = short_conv(quant(h @ w(p + "q").T), w(p + "q.conv"))
    k, _ = short_conv(quant(h @ w(p + "k").T), w(p + "k.conv"))
    v, _ = short_conv(quant(h @ w(p + "v").T), w(p + "v.conv"))
    q, k, v = silu(q).view(t, kv, dim), silu(k).view(t, kv, dim), silu(v).view(t, heads, vdim)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(group, dim=1), k.repeat_interleave(group, dim=1)
    beta = torch.sigmoid(quant(h @ w(p + "b").T))
    g = torch.exp(-torch.exp(w(p + "A_log")) * softplus(quant(h @ w(p + "a").T) + w(p + "dt_bias")))
    o, _ = delta_rule(q, k, v, beta, g)
    o = norm_plain(o, w(p + "norm"), eps).reshape(t, heads * vdim) * silu(quant(h @ w(p + "g").T))
    return quant(o) @ w(p + "o").T


# ---------------------------------------------------------------------------------------------- feed-forwards

def dense_ff(h, w, p, quant=no_quant):
    return quant(torch.relu(h @ w(p + "gate").T) * (h @ w(p + "up").T)) @ w(p + "down").T


def expert_ff(h, w, p, mlp, quant=no_quant):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    ids, weights = route_softmax(h @ w(p + "router").T, top)
    out = torch.zeros_like(h)
    for e in range(n):
        y = quant(silu(h @ w(p + f"e{e}.gate").T) * (h @ w(p + f"e{e}.up").T)) @ w(p + f"e{e}.down").T
        for c in range(top):
            out = out + torch.where((ids[:, c] == e)[:, None], weights[:, c][:, None] * y, torch.zeros_like(y))
    return out


# ---------------------------------------------------------------------------------------------- the model

def forward(cfg, weights, tokens, dtype=torch.float64, quant=no_quant, layers_out=None):
    """Logits [T, vocab] of one whole sequence; `layers_out` (a list) receives the stream after every layer."""
    def w(name):
        return weights[name].to(dtype)
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tokens.numel())
    x = w("embed")[tokens] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = quant(norm_one_plus(x, w(p + "norm1"), eps))
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = attention_mixer(h, w, p + "mix.", m, eps, pos, quant)
        elif kind == "latent_attention":
            y = latent_attention_mixer(h, w, p + "mix.", m, eps, pos, quant)
        elif kind == "delta":
            y = delta_mixer(h, w, p + "mix.", m, eps, quant)
        else:
            raise ValueError(kind)
        x = x + norm_one_plus(y, w(p + "norm1b"), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = quant(norm_one_plus(x, w(p + "norm2"), eps))
            y = dense_ff(h, w, p + "mlp.", quant) if mlp["kind"] == "dense" else expert_ff(h, w, p + "mlp.", mlp, quant)
            x = x + norm_one_plus(y, w(p + "norm2b"), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = quant(norm_one_plus(x, w("final.norm"), eps))
    return h @ w("head").T
