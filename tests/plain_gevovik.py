"""A plain, slow implementation of the Gevovik decoder, one function per mechanism, written from the design's
equations and sharing no code with the package.  Everything is torch on the CPU in the dtype it is asked for
(float64 for an oracle); recurrences are walked token by token and attention is a full score matrix.

The design.  x_t = embed[tok_t] * s + bigram[(tok_(t-1) * a + tok_t * b) mod n]  (row n for a sequence's first token).
A layer norms what a branch gives, not what it reads:
    x += n1(mixer(x));   x += n2(ff(x))          n(y) = y / sqrt(mean(y^2) + eps) * g,  g ONE learned number
(no second line when the layer has no feed-forward).  Mixers:
  mamba2            [z | x | B | C | dt] = Win h; x, B, C through a short causal convolution with bias and silu;
                    dt = softplus(dt + bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x;
                    (y * silu(z)) normed in equal parts, times a weight; Wo.
  latent_attention  keys and values are projections of one small normed latent per token plus one rotated key part
                    shared by the heads; queries are [plain | rotated] per head; neighbours (2i, 2i + 1) are rotated;
                    causal softmax whose denominator also holds exp(sink_h); Wo.  A layer may use the latent and the
                    rotated key part of an earlier layer instead of making its own.
  parallel          ls * left(h) + rs * right(h):
      left          grouped heads, q and k normed per head, the first dims of every head rotated in halves
                    (i, i + dims/2) with stretched frequencies; scores times a number per head, then mixed across heads
                    by a matrix, a window of the last n keys, softmax, head h times sigmoid(Wg h)_h, Wo.
      right         the gated delta rule with a decay per key channel: q, k, v through convolutions and silu, q and k
                    unit vectors (q also / sqrt(dim)); S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q;
                    o / rms(o) * w * sigmoid(Wg2 Wg1 h); Wo.
Feed-forward: Wd relu(Wu h)^2.  Output: the model's norm, then the head matrix."""
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


def scalar_norm(x, g, eps):
    """The layer norm of the design: one learned number for all coordinates."""
    return rms_unit(x, eps) * g


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.clamp(x, min=0) + torch.log1p(torch.exp(-x.abs()))


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table per token; the first token of a sequence takes the table's last row."""
    rows = [buckets]
    for p, c in zip(tokens[:-1], tokens[1:]):
        rows.append((p * mul_prev + c * mul_cur) % buckets)
    return rows


def short_conv(x, taps, bias=None):
    """y[t, c] = sum_j taps[c, j] x[t - (n - 1) + j, c] (+ bias[c]), zeros before the start."""
    n = taps.shape[1]
    pad = torch.cat([x.new_zeros(n - 1, x.shape[1]), x], dim=0)
    y = sum(pad[j: j + x.shape[0]] * taps[:, j] for j in range(n))
    return y if bias is None else y + bias


def rotation_frequencies(dims, base, scaling=None, dtype=torch.float64):
    """f_i = base^(-2i / dims); with scaling, a blend of f_i / factor and f_i by a ramp over the pair index, and the
    factor both cos and sin are multiplied by."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    mag = 1.0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def turn_dim(turns):
            return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    return f.to(dtype), mag


def rotate(x, positions, freq, mag, dims, layout):
    """x [T, heads, d]: the first `dims` values of every head turn by positions * freq; layout "halves" pairs value i
    with i + dims/2, "pairs" value 2i with 2i + 1."""
    ang = positions.to(freq.dtype)[:, None] * freq[None, :]
    c, s = (torch.cos(ang) * mag).to(x.dtype)[:, None, :], (torch.sin(ang) * mag).to(x.dtype)[:, None, :]
    out = x.clone()
    half = dims // 2
    if layout == "halves":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half], out[..., half:dims] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    return out


def masked_softmax_attention(scores, v, window=None, sink=None):
    """scores [H, T, T] (query, key), v [H, T, vd]: causal (and the last `window` keys only), softmax over the
    visible keys; with `sink` [H] the denominator also holds exp(sink_h)."""
    t = scores.shape[1]
    i, j = torch.arange(t)[:, None], torch.arange(t)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    scores = scores.masked_fill(~seen, float("-inf"))
    if sink is not None:
        col = sink.to(scores.dtype)[:, None, None].expand(-1, t, 1)
        p = torch.softmax(torch.cat([scores, col], dim=-1), dim=-1)[..., :t]
    else:
        p = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,hjd->ihd", p, v)


def delta_rule_channel_decay(q, k, v, g, beta):
    """q, k [T, H, kd], v [T, H, vd], g [T, H, kd], beta [T, H]: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q, token by token from a zero state."""
    t, h, kd = q.shape
    s = q.new_zeros(h, kd, v.shape[2])
    out = []
    for n in range(t):
        s = s * g[n][:, :, None]
        u = beta[n][:, None] * (v[n] - torch.einsum("hkv,hk->hv", s, k[n]))
        s = s + k[n][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", s, q[n]))
    return torch.stack(out)


def state_space_scan(x, b, c, decay, dt):
    """x [T, H, vd], b, c [T, H, N], decay, dt [T, H]: S <- decay S + dt b x^T; y = S^T c."""
    t, h, vd = x.shape
    s = x.new_zeros(h, b.shape[2], vd)
    out = []
    for n in range(t):
        s = s * decay[n][:, None, None] + (dt[n][:, None] * b[n])[:, :, None] * x[n][:, None, :]
        out.append(torch.einsum("hnv,hn->hv", s, c[n]))
    return torch.stack(out)


# ---------------------------------------------------------------------------------------------- mixers

def mamba2(m, w, p, h, eps, quant):
    heads, vd, n, groups, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = heads * vd
    proj = quant(h @ w[p + "in"].T)
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
    xbc = silu(short_conv(xbc, w[p + "conv"].to(h.dtype), w[p + "conv.b"].to(h.dtype)))
    t = h.shape[0]
    x = xbc[:, :inner].view(t, heads, vd)
    per = heads // groups
    b = xbc[:, inner: inner + groups * n].view(t, groups, n).repeat_interleave(per, dim=1)
    c = xbc[:, inner + groups * n:].view(t, groups, n).repeat_interleave(per, dim=1)
    dt = softplus(dt + w[p + "dt_bias"].to(h.dtype))
    decay = torch.exp(-torch.exp(w[p + "A_log"].to(h.dtype)) * dt)
    y = state_space_scan(x, b, c, decay, dt) + w[p + "D"].to(h.dtype)[None, :, None] * x
    y = (y.reshape(t, inner) * silu(z)).view(t, parts, inner // parts)
    y = quant(rms_unit(y, eps).reshape(t, inner) * w[p + "norm"].to(h.dtype))
    return y @ w[p + "o"].T


def latent_parts(m, w, p, h, positions, eps, quant):
    """What a latent attention caches per token: the normed latent and the rotated key part."""
    rank, rd = m["kv_rank"], m["rot_dim"]
    dkv = quant(h @ w[p + "dkv"].T)
    c = quant(rms_unit(dkv[:, :rank], eps) * w[p + "dkv.norm"].to(h.dtype))
    freq, mag = rotation_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"), h.dtype)
    kr = quant(rotate(dkv[:, None, rank:], positions, freq, mag, m["rot"]["dims"], "pairs")[:, 0])
    return c, kr


def latent_attention(m, w, p, h, positions, eps, quant, shared=None):
    heads, nd, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    t = h.shape[0]
    c, kr = shared if shared is not None else latent_parts(m, w, p, h, positions, eps, quant)
    q = quant(h @ w[p + "q"].T).view(t, heads, nd + rd)
    freq, mag = rotation_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"), h.dtype)
    q_rot = quant(rotate(q[..., nd:], positions, freq, mag, m["rot"]["dims"], "pairs"))
    k_plain = (c @ w[p + "uk"].T).view(t, heads, nd)
    v = (c @ w[p + "uv"].T).view(t, heads, vd)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :nd], k_plain) + torch.einsum("ihd,jd->hij", q_rot, kr)) * m["scale"]
    o = masked_softmax_attention(scores, v.transpose(0, 1), sink=w[p + "sink"])
    return quant(o.reshape(t, heads * vd)) @ w[p + "o"].T, (c, kr)


def talking_window_attention(m, w, p, h, positions, eps, quant):
    heads, kvh, kd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = quant(h @ w[p + "q"].T).view(t, heads, kd)
    k = quant(h @ w[p + "k"].T).view(t, kvh, kd)
    v = quant(h @ w[p + "v"].T).view(t, kvh, vd)
    q = rms_unit(q, eps) * w[p + "q.norm"].to(h.dtype)
    k = rms_unit(k, eps) * w[p + "k.norm"].to(h.dtype)
    if m.get("rot"):
        freq, mag = rotation_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"), h.dtype)
        q, k = (rotate(x, positions, freq, mag, m["rot"]["dims"], "halves") for x in (q, k))
    q, k = quant(q), quant(k)
    per = heads // kvh
    scores = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(per, dim=1)) * m["scale"]
    scores = scores * w[p + "temp"].to(h.dtype)[:, None, None]
    scores = torch.einsum("hg,gij->hij", w[p + "talk"].to(h.dtype), scores)
    o = masked_softmax_attention(scores, v.repeat_interleave(per, dim=1).transpose(0, 1), window=(m.get("mask") or {}).get("size"))
    gate = torch.sigmoid(quant(h @ w[p + "g"].T))
    return quant((o * gate[:, :, None]).reshape(t, heads * vd)) @ w[p + "o"].T


def channel_delta(m, w, p, h, eps, quant):
    heads, kvh, kd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    per = heads // kvh

    def conv(name):
        return silu(short_conv(quant(h @ w[p + name].T), w[p + name + ".conv"].to(h.dtype)))
    q, k, v = conv("q").view(t, kvh, kd), conv("k").view(t, kvh, kd), conv("v").view(t, heads, vd)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * kd ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(per, dim=1), k.repeat_interleave(per, dim=1)
    beta = torch.sigmoid(quant(h @ w[p + "b"].T))
    a = quant(h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"].to(h.dtype)
    g = torch.exp(-torch.exp(w[p + "A_log"].to(h.dtype))[None, :, None] * softplus(a).view(t, heads, kd))
    o = delta_rule_channel_decay(q, k, v, g, beta)
    gate = torch.sigmoid(quant(quant(h @ w[p + "g1"].T) @ w[p + "g2"].T)).view(t, heads, vd)
    y = quant(rms_unit(o, eps) * w[p + "norm"].to(h.dtype) * gate)
    return y.reshape(t, heads * vd) @ w[p + "o"].T


def parallel(m, w, p, h, positions, eps, quant):
    left = talking_window_attention(m["left"], w, p + "left.", h, positions, eps, quant)
    right = channel_delta(m["right"], w, p + "right.", h, eps, quant)
    return m["left_scale"] * left + m["right_scale"] * right


def feed_forward(mlp, w, p, h, quant):
    a = torch.relu(h @ w[p + "up"].T)
    return quant(a * a) @ w[p + "down"].T


# ---------------------------------------------------------------------------------------------- the model

def forward(cfg, weights, tokens, dtype=torch.float64, quant=no_quant, streams=None):
    """Logits [T, vocab] of one sequence.  `streams`: a list that receives the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(tok))
    x = w["embed"][tok] * cfg["embedding"]["scale"]
    big = cfg["embedding"].get("bigram")
    if big:
        rows = bigram_rows(list(tokens), big["buckets"], big["mul_prev"], big["mul_cur"])
        x = x + w["bigram"][torch.as_tensor(rows)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        h = quant(x)
        if layer["type"] == "mamba2":
            y = mamba2(m, w, p, h, eps, quant)
        elif layer["type"] == "latent_attention":
            y, kept[i] = latent_attention(m, w, p, h, positions, eps, quant,
                                          shared=kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif layer["type"] == "parallel":
            y = parallel(m, w, p, h, positions, eps, quant)
        else:
            raise ValueError(layer["type"])
        x = x + scalar_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + scalar_norm(feed_forward(layer["mlp"], w, f"l{i}.mlp.", quant(x), quant), w[f"l{i}.norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return quant(scalar_norm(x, w["final.norm"], eps)) @ w["head"].T
