"""Tiny Fiponex configurations for the tests and the plain implementation's logits for them.

The configurations differ from one another in every size and option: widths, head counts and grouping, key size
against value size (equal in one layer only), sizes the tensor-core kernels take and sizes that are multiples of
nothing convenient, windows that are and are not multiples of the page (one shorter than a page, one absent), a query
stretch that starts at position 0 / late / never, rotation over the whole rotated part and over half of it, filters of
1, 2, 3 and 4 taps, one query/key head per value head and one for all, layers without a feed-forward, every expert
chosen / one chosen, an embedding scale of 1, and the order of the layer kinds (a model of recurrent layers only
keeps no keys at all), and head groups larger than four.  Pages of 4, 8, 16 and 32 tokens."""
import torch

import plain_fiponex as pf


def attention(heads, kv, dim, vdim, scale, q_temp=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, size=None, rot=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if size:
        m["mask"] = {"size": size}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def delta(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def model(vocab, width, scale, eps, init, layers):
    return {"architecture": "Fiponex", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "initializer_range": init, "layers": layers}


# sizes the bfloat16 tensor-core kernels take (keys and values in multiples of 16, widths in multiples of 8)
FIP_A = model(211, 64, 8.0, 1e-5, 0.1, [
    attention(4, 2, 16, 32, 0.3, q_temp=(0.4, 8), mlp=dense(96)),
    latent(3, 16, 16, 24, 32, 0.2, size=20, rot=(16, 100.0), mlp=moe(6, 2, 40)),
    delta(4, 2, 16, 8, 4),
    latent(2, 8, 16, 16, 48, 0.15, size=37, rot=(16, 5000.0), mlp=dense(72)),
])
FIP_B = model(331, 96, 3.5, 1e-6, 0.08, [
    delta(3, 3, 24, 40, 2, mlp=moe(3, 3, 56)),
    attention(3, 1, 32, 16, 0.2, mlp=moe(9, 4, 24)),
    latent(2, 24, 16, 40, 40, 0.25, size=33, rot=(8, 2000.0)),
    attention(6, 6, 16, 16, 0.35, q_temp=(1.0, 40), mlp=dense(40)),
    delta(6, 1, 32, 16, 3, mlp=dense(64)),
])
# sizes that are multiples of nothing convenient; a window shorter than the page; no window at all; one tap
FIP_C = model(128, 44, 1.0, 1e-4, 0.15, [
    latent(5, 6, 10, 14, 18, 0.4, size=3, rot=(10, 30.0), mlp=moe(7, 1, 12)),
    attention(6, 3, 10, 6, 0.5, q_temp=(0.25, 1), mlp=None),
    latent(1, 12, 4, 6, 9, 0.3, rot=(2, 10.0), mlp=dense(20)),
    delta(2, 1, 6, 10, 1, mlp=moe(2, 2, 6)),
])
# recurrent layers only: the cache manager has no page pool to run
FIP_D = model(97, 40, 2.0, 1e-5, 0.12, [
    delta(2, 2, 10, 14, 4, mlp=dense(24)),
    delta(5, 1, 8, 8, 2, mlp=None),
])
# head groups of 8 and 5 (more query heads per key/value head than a kernel handles in one pass), a long key row
# beside a short value row, a latent whose cached row is far longer than any head's, a window of hundreds, seven layers.
# Its requests are long, so every routed layer chooses all its experts: among hundreds of tokens one always has two
# experts' scores closer than bfloat16 rounding, and which of the two is taken is not what this configuration is for.
FIP_E = model(257, 128, 11.3, 1e-6, 0.05, [
    attention(8, 1, 80, 48, 0.11, q_temp=(0.5, 64), mlp=moe(5, 5, 32)),
    latent(8, 32, 16, 48, 64, 0.15, size=150, rot=(16, 250000.0), mlp=dense(160)),
    delta(8, 2, 48, 32, 4, mlp=moe(4, 4, 48)),
    attention(10, 2, 16, 64, 0.25, mlp=dense(96)),
    delta(2, 2, 64, 96, 3, mlp=dense(64)),
    latent(4, 48, 32, 16, 96, 0.1, size=129, rot=(32, 10000.0), mlp=moe(8, 8, 16)),
    attention(2, 2, 128, 128, 0.09, q_temp=(0.2, 100), mlp=None),
])
FIP = {"A": (FIP_A, 16, 3), "B": (FIP_B, 8, 4), "C": (FIP_C, 4, 5), "D": (FIP_D, 4, 6), "E": (FIP_E, 32, 9)}   # config, page size, seed


def write_models(tmp_path_factory):
    from tiny_llm_b200.config import FiponexConfig
    from tiny_llm_b200.weights import write_random_model

    out = {}
    for name, (cfg, _page, seed) in FIP.items():
        d = tmp_path_factory.mktemp(f"fip_{name}")
        write_random_model(str(d), FiponexConfig.from_dict(cfg), seed=seed, dtype=torch.float32)
        out[name] = str(d)
    return out


def plain_model(model_dir, dtype):
    """Configuration, weights and storage rounding of the plain implementation for one of the engine's two paths."""
    cfg, w = pf.load_config(model_dir), pf.load_weights(model_dir)
    if dtype == "bfloat16":   # matrices are held in the engine's dtype, small vectors in 32-bit
        w = {k: (v if v.dim() < 2 or k.endswith(".conv") else v.to(torch.bfloat16).float()) for k, v in w.items()}
    return cfg, w, (pf.no_quant if dtype == "float32" else pf.bf16_quant)


def plain_logits(model_dir, reqs, dtype):
    """What the engine's logits are held against: the plain implementation in 64-bit with the path's weights (rounded
    to bfloat16 for the bfloat16 path) and NO rounding of activations, i.e. the result the path approximates."""
    cfg, w, _ = plain_model(model_dir, dtype)
    return {rid: pf.forward(cfg, w, toks, torch.float64).float() for rid, toks in reqs.items()}


def tolerances(model_dir, reqs, dtype):
    """Per request, how far the engine may be from the plain implementation's 64-bit logits.  32-bit: 2e-5, or four
    times what 32-bit rounding does to the plain implementation itself where that is more.  bfloat16: twice what
    bfloat16 rounding of the activations does to the plain implementation for this very request.  The engine rounds
    at the same places but sums in another order, so its error is another draw of the same size.  (A fault -- a
    wrong key, a lost state, a window edge off by one -- is caught by the 32-bit runs of the same code.)"""
    out = {}
    for rid, toks in reqs.items():
        cfg, w, quant = plain_model(model_dir, dtype)
        f64 = pf.forward(cfg, w, toks, torch.float64)
        if dtype == "float32":
            f32 = pf.forward(cfg, w, toks, torch.float32)
            out[rid] = max(2e-5, 4.0 * float((f32.double() - f64).abs().max()))
        else:
            out[rid] = 2.0 * float((pf.forward(cfg, w, toks, torch.float64, quant=quant) - f64).abs().max())
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
