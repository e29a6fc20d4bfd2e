"""Tiny Gevovik configurations for the tests and the plain implementation's logits for them.

The configurations differ from one another in every size and option: widths, head counts and grouping (one key/value
head per query head, one for all, some), key size against value size, rotation over a whole head and over part of it,
with and without stretched frequencies, windows shorter than a page, longer than several pages, and absent, filters of
1 to 4 taps, state-space groups of 1 / some / all heads, norm parts that are and are not whole heads, a latent layer
that reads another layer's cache (directly behind it, and several layers on), layers without a feed-forward, a model
without bigram rows, a single bucket, an embedding scale of 1, recurrent layers only (no page pool at all), sizes the
tensor-core kernels take and sizes that are multiples of nothing convenient.  Pages of 4, 8, 16 and 32 tokens."""
import torch

import plain_gevovik as pg


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def mamba2(heads, vdim, state, groups, parts, conv, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": parts, "conv": conv}}


def latent(heads, dim, rot_dim, vdim, rank, scale, r, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": r}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def parallel(left, right, ls, rs, mlp=None):
    heads, kv, dim, vdim, scale, size, r = left
    lm = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        lm["mask"] = {"size": size}
    if r:
        lm["rot"] = r
    rm = dict(zip(("heads", "kv_heads", "dim", "vdim", "conv"), right))
    return {"type": "parallel", "mixer": {"left": lm, "right": rm, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model(vocab, width, scale, bigram, eps, init, layers):
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return {"architecture": "Gevovik", "vocab": vocab, "width": width, "embedding": emb, "norm": {"eps": eps},
            "initializer_range": init, "layers": layers}


# sizes the bfloat16 tensor-core kernels take (keys and values in multiples of 16, widths in multiples of 8)
GEV_A = model(211, 64, 8.0, (97, 7, 13), 1e-5, 0.1, [
    parallel((4, 2, 16, 32, 0.3, 20, rot(16, 100.0, (2.0, 16, 4.0, 1.0))), (4, 2, 16, 8, 4), 0.7, 1.3, mlp=dense(96)),
    latent(3, 16, 16, 24, 32, 0.2, rot(16, 100.0), mlp=dense(72)),
    mamba2(4, 16, 16, 2, 2, 4),
    latent(2, 8, 16, 16, 32, 0.15, rot(16, 100.0), kv_from=1, mlp=dense(40)),
])
# sizes that are multiples of nothing convenient; a window shorter than the page; no window; no rotation; one tap;
# no bigram rows; norm parts that cut through heads
GEV_B = model(128, 44, 1.0, None, 1e-4, 0.15, [
    mamba2(6, 6, 10, 3, 4, 2, mlp=dense(20)),
    parallel((6, 3, 10, 6, 0.5, 3, rot(6, 30.0)), (2, 1, 6, 10, 1), 1.0, 0.4),
    latent(5, 6, 10, 14, 18, 0.4, rot(10, 30.0, (3.0, 8, 2.0, 0.5)), mlp=dense(12)),
    parallel((2, 2, 12, 12, 0.3, None, None), (3, 3, 8, 8, 3), 0.25, 2.0, mlp=dense(28)),
    latent(1, 12, 10, 6, 18, 0.3, rot(10, 30.0, (3.0, 8, 2.0, 0.5)), kv_from=2),
])
# recurrent layers only: the cache manager has no page pool to run; one bucket; groups of one head and of all heads
GEV_C = model(97, 40, 2.0, (1, 3, 5), 1e-5, 0.12, [
    mamba2(5, 8, 12, 5, 1, 3, mlp=dense(24)),
    mamba2(2, 20, 7, 1, 5, 1),
    mamba2(4, 10, 16, 2, 40, 4, mlp=dense(16)),
])
# larger: head groups of 4 and 8, windows of hundreds over many pages, a rotation stretched past a short original
# length, a latent far longer than any head, two layers reading one layer's cache, seven layers
GEV_D = model(257, 128, 11.3, (509, 1000003, 31), 1e-6, 0.05, [
    latent(8, 32, 16, 48, 64, 0.15, rot(16, 300000.0, (8.0, 64, 16.0, 2.0)), mlp=dense(160)),
    parallel((8, 2, 32, 16, 0.18, 150, rot(32, 10000.0, (4.0, 64, 8.0, 1.0))), (8, 2, 48, 32, 4), 0.8, 0.9, mlp=dense(96)),
    mamba2(8, 32, 64, 2, 1, 4, mlp=dense(64)),
    latent(4, 48, 16, 16, 64, 0.1, rot(16, 300000.0, (8.0, 64, 16.0, 2.0)), kv_from=0),
    parallel((8, 1, 64, 64, 0.12, 129, rot(16, 500.0)), (2, 2, 64, 96, 3), 1.5, 0.5, mlp=dense(64)),
    mamba2(16, 8, 32, 16, 4, 2),
    latent(2, 16, 16, 80, 64, 0.2, rot(16, 300000.0, (8.0, 64, 16.0, 2.0)), kv_from=0, mlp=dense(48)),
])
GEV = {"A": (GEV_A, 16, 3), "B": (GEV_B, 4, 4), "C": (GEV_C, 8, 5), "D": (GEV_D, 32, 9)}   # config, page size, seed


def write_models(tmp_path_factory):
    from tiny_llm_b200.config import GevovikConfig
    from tiny_llm_b200.weights import write_random_model

    out = {}
    for name, (cfg, _page, seed) in GEV.items():
        d = tmp_path_factory.mktemp(f"gev_{name}")
        write_random_model(str(d), GevovikConfig.from_dict(cfg), seed=seed, dtype=torch.float32)
        out[name] = str(d)
    return out


def plain_model(model_dir, dtype):
    """Configuration, weights and storage rounding of the plain implementation for one of the engine's two paths."""
    cfg, w = pg.load_config(model_dir), pg.load_weights(model_dir)
    if dtype == "bfloat16":   # matrices are held in the engine's dtype; vectors, filters and the heads' mixing in 32-bit
        w = {k: (v if v.dim() < 2 or k.endswith(".conv") or k.endswith(".talk") else v.to(torch.bfloat16).float())
             for k, v in w.items()}
    return cfg, w, (pg.no_quant if dtype == "float32" else pg.bf16_quant)


def plain_logits(model_dir, reqs, dtype):
    """What the engine's logits are held against: the plain implementation in 64-bit with the path's weights (rounded
    to bfloat16 for the bfloat16 path) and NO rounding of activations, i.e. the result the path approximates."""
    cfg, w, _ = plain_model(model_dir, dtype)
    return {rid: pg.forward(cfg, w, toks, torch.float64).float() for rid, toks in reqs.items()}


def tolerances(model_dir, reqs, dtype):
    """Per request, how far the engine may be from the plain implementation's 64-bit logits.  32-bit: 2e-5, or four
    times what 32-bit rounding does to the plain implementation itself where that is more.  bfloat16: twice what
    bfloat16 rounding of the activations does to the plain implementation for this very request.  The engine rounds
    at the same places but sums in another order, so its error is another draw of the same size.  (A fault -- a
    wrong key, a lost state, a window edge off by one -- is caught by the 32-bit runs of the same code.)"""
    out = {}
    for rid, toks in reqs.items():
        cfg, w, quant = plain_model(model_dir, dtype)
        f64 = pg.forward(cfg, w, toks, torch.float64)
        if dtype == "float32":
            f32 = pg.forward(cfg, w, toks, torch.float32)
            out[rid] = max(2e-5, 4.0 * float((f32.double() - f64).abs().max()))
        else:
            out[rid] = 2.0 * float((pg.forward(cfg, w, toks, torch.float64, quant=quant) - f64).abs().max())
    return out


def compare(got, ref, prefix, tol, what):
    worst = 0.0
    for rid, r in ref.items():
        g = got[prefix + rid]
        assert g.shape == r.shape, (what, rid, g.shape, r.shape)
        diff = (g - r).abs()
        if not float(diff.max()) <= tol[rid]:
            bad = (~(diff.max(dim=1).values <= tol[rid])).nonzero().flatten()
            raise AssertionError(f"{what}: request {rid} differs from the plain implementation first at position "
                                 f"{int(bad[0])} of {r.shape[0]} (max |diff| {float(diff.max()):.3e}, tolerance "
                                 f"{tol[rid]:.3e}; wrong positions: {bad.tolist()[:20]})")
        worst = max(worst, float(diff.max()) / tol[rid])
    import replay_util
    replay_util.record_margin(what, "", worst)   # printed, and appended to the file TLLM_MARGIN_FILE names
    return worst
