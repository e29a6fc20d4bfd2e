"""Fiponex on the host: the configuration and its errors, tensor names, cache needs, the block's parts, and the plain
implementation against closed forms and against itself (the latent attention taken against the cached latent equals
the one with keys and values written out; filters and the delta rule carried over a cut)."""
import copy

import pytest
import torch

import plain_fiponex as pf
from fiponex_util import FIP, FIP_A, FIP_B, FIP_C, FIP_D


def test_config_round_trip_and_registry():
    from tiny_llm_b200.config import FiponexConfig, config_from_dict
    for cfg, _, _ in FIP.values():
        c = config_from_dict(cfg)
        assert isinstance(c, FiponexConfig)
        again = FiponexConfig.from_dict(c.to_dict())
        assert again == c
        spec = c.model_spec()
        assert spec.embedding_scale == cfg["embedding"]["scale"] and len(spec.layers) == len(cfg["layers"])
        assert all(l.block == "sandwich_norm" for l in spec.layers)


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mixer", "scale"), None, "scale"),
    (("layers", 0, "mixer", "q_temp", "every"), 0, "every"), (("layers", 1, "mixer", "kv_rank"), -1, "kv_rank"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "dims"), (("layers", 1, "mixer", "rot", "dims"), 18, "dims"),
    (("layers", 1, "mlp", "router", "top"), 9, "top"), (("layers", 2, "mixer", "conv"), 0, "conv"),
    (("layers", 2, "type"), "mamba", "mamba"), (("layers", 0, "mlp", "kind"), "sparse", "sparse"),
    (("norm",), None, "norm"), (("vocab",), 0, "vocab")])
def test_config_errors_name_the_key(path, value, word):
    from tiny_llm_b200.config import ConfigError, FiponexConfig
    cfg = copy.deepcopy(FIP_A)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        FiponexConfig.from_dict(cfg)
    assert word in str(e.value)


def test_tensor_names_and_shapes():
    from tiny_llm_b200.config import FiponexConfig
    from tiny_llm_b200.parts import DecoderModel
    specs = DecoderModel(FiponexConfig.from_dict(FIP_A).model_spec()).weight_specs()
    want = {"embed": (211, 64), "head": (211, 64), "final.norm": (64,), "l0.norm1": (64,), "l0.norm1b": (64,), "l0.norm2b": (64,),
            "l0.mix.q": (64, 64), "l0.mix.q.b": (64,), "l0.mix.k": (32, 64), "l0.mix.v": (64, 64), "l0.mix.v.b": (64,),
            "l0.mix.q.norm": (16,), "l0.mix.k.norm": (16,), "l0.mix.sink": (4,), "l0.mix.g": (128, 64), "l0.mix.o": (64, 128),
            "l0.mlp.gate": (96, 64), "l0.mlp.down": (64, 96),
            "l1.mix.q": (96, 64), "l1.mix.dkv": (48, 64), "l1.mix.dkv.norm": (32,), "l1.mix.uk": (48, 32), "l1.mix.uv": (72, 32),
            "l1.mix.sink": (3,), "l1.mix.g": (3, 64), "l1.mix.o": (64, 72), "l1.mlp.router": (6, 64), "l1.mlp.e5.gate": (40, 64),
            "l1.mlp.e0.down": (64, 40),
            "l2.mix.q": (32, 64), "l2.mix.q.conv": (32, 4), "l2.mix.v": (32, 64), "l2.mix.v.conv": (32, 4), "l2.mix.b": (4, 64),
            "l2.mix.a": (4, 64), "l2.mix.A_log": (4,), "l2.mix.dt_bias": (4,), "l2.mix.norm": (8,), "l2.mix.g": (32, 64),
            "l2.mix.o": (64, 32)}
    for name, shape in want.items():
        assert name in specs and tuple(specs[name].shape) == shape, name
    assert "l2.norm2" not in specs and "l2.norm2b" not in specs and "l1.mlp.correction" not in specs     # no feed-forward there


def test_cache_needs():
    from tiny_llm_b200.cache import CacheManager, KVNeed, StateNeed
    from tiny_llm_b200.config import FiponexConfig
    from tiny_llm_b200.parts import DecoderModel
    needs = DecoderModel(FiponexConfig.from_dict(FIP_A).model_spec()).cache_needs()
    assert needs[0] == KVNeed(2, 16, None, value_dim=32)
    assert needs[1] == KVNeed(1, 48, 20, value_dim=32)          # one shared row: [latent | rotated part], value = latent
    assert needs[2] == (StateNeed((4, 8, 16), torch.float32), StateNeed((3, 96), torch.float32))
    assert needs[3] == KVNeed(1, 64, 37, value_dim=48)
    cache = CacheManager(needs, max_tokens=256, page_size=16, max_slots=4)
    assert len(cache.groups) == 3 and len(cache.slots.needs) == 2
    # a model of recurrent layers only keeps no keys
    only = CacheManager(DecoderModel(FiponexConfig.from_dict(FIP_D).model_spec()).cache_needs(), 64, 4, 4)
    assert only.groups == [] and len(only.slots.needs) == 4
    only.add_request("a")
    assert only.reserve("a", 50)
    only.commit("a", 50)
    only.free_request("a")
    only.check()


def test_pages_behind_a_window_go_back_and_slots_are_used_again():
    from tiny_llm_b200.cache import CacheManager
    from tiny_llm_b200.config import FiponexConfig
    from tiny_llm_b200.parts import DecoderModel
    cache = CacheManager(DecoderModel(FiponexConfig.from_dict(FIP_A).model_spec()).cache_needs(), 128, 16, 2)
    assert cache.add_request("a") is not None and cache.add_request("b") is not None and cache.add_request("c") is None
    for n in (5, 60, 1, 1, 30):
        assert cache.reserve("a", n)
        cache.commit("a", n)
        cache.check()
    by_window = {g.need.window: g for g in cache.groups}
    assert by_window[None].pool.num_used == -(-97 // 16)
    assert by_window[20].pool.num_used == 97 // 16 - (97 - 20 + 1) // 16 + 1
    cache.free_request("a")
    assert cache.add_request("c") is not None
    assert all(g.pool.num_used == 0 for g in cache.groups)


def test_the_block_norms_both_sides_of_each_branch():
    from tiny_llm_b200.config import FiponexConfig
    from tiny_llm_b200.parts import DecoderModel, SandwichBlock
    model = DecoderModel(FiponexConfig.from_dict(FIP_C).model_spec())
    assert all(isinstance(b, SandwichBlock) for b in model.blocks)
    assert len(model.blocks[0].parts()) == 6 and len(model.blocks[1].parts()) == 3 and model.graph_safe
    assert all(n.one_plus for n in (model.final_norm, model.blocks[0].norm1, model.blocks[0].norm2_out))


def test_plain_softmax_with_a_sink_against_the_closed_form():
    q = torch.tensor([[[1.0, 0.0]]], dtype=torch.float64)
    k = torch.tensor([[[2.0, 0.0]], [[0.0, 5.0]], [[1.0, 1.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[10.0]], [[100.0]]], dtype=torch.float64)
    sink = torch.tensor([0.7], dtype=torch.float64)
    out = pf.sink_softmax_attention(q, k, v, torch.tensor([2]), torch.arange(3), 0.5, sink)
    e = torch.exp(torch.tensor([1.0, 0.0, 0.5], dtype=torch.float64))
    assert abs(float(out) - float((e * torch.tensor([1.0, 10.0, 100.0])).sum() / (e.sum() + torch.exp(sink[0])))) < 1e-12
    out = pf.sink_softmax_attention(q, k, v, torch.tensor([2]), torch.arange(3), 0.5, sink, window=2)   # key 0 has left
    assert abs(float(out) - float((e[1] * 10 + e[2] * 100) / (e[1] + e[2] + torch.exp(sink[0])))) < 1e-12
    out = pf.sink_softmax_attention(q, k, v, torch.tensor([0]), torch.arange(3), 0.5, sink)             # causal
    assert abs(float(out) - float(e[0] / (e[0] + torch.exp(sink[0])))) < 1e-12


def test_latent_attention_against_the_cached_latent_equals_the_written_out_form():
    """What the engine computes: with q' = Wuk^T q_plain the scores are q' . c + q_rot . k_rot, the weighted sum is
    taken over the latents, and the head's value projection comes last."""
    g = torch.Generator().manual_seed(1)
    t, heads, nd, rd, vd, rank, scale, window = 40, 3, 6, 4, 5, 9, 0.3, 7
    q = torch.randn(t, heads, nd + rd, generator=g, dtype=torch.float64)
    c = torch.randn(t, rank, generator=g, dtype=torch.float64)
    k_rot = torch.randn(t, 1, rd, generator=g, dtype=torch.float64)
    uk = torch.randn(heads * nd, rank, generator=g, dtype=torch.float64)
    uv = torch.randn(heads * vd, rank, generator=g, dtype=torch.float64)
    sink = torch.randn(heads, generator=g, dtype=torch.float64)
    pos = torch.arange(t)
    k = torch.cat([(c @ uk.T).view(t, heads, nd), k_rot.expand(t, heads, rd)], dim=-1)
    direct = pf.sink_softmax_attention(q, k, (c @ uv.T).view(t, heads, vd), pos, pos, scale, sink, window)
    q_lat = torch.cat([torch.einsum("thd,hdr->thr", q[..., :nd], uk.view(heads, nd, rank)), q[..., nd:]], dim=-1)
    shared_k = torch.cat([c, k_rot[:, 0]], dim=-1).view(t, 1, rank + rd)
    o_lat = pf.sink_softmax_attention(q_lat, shared_k, c.view(t, 1, rank), pos, pos, scale, sink, window)
    absorbed = torch.einsum("thr,hvr->thv", o_lat, uv.view(heads, vd, rank))
    assert float((direct - absorbed).abs().max()) < 1e-12


def test_pairwise_rotation_keeps_lengths_and_relative_angles():
    g = torch.Generator().manual_seed(2)
    x, y = torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    def dot(p, r):
        return float((pf.rotate_pairs(x, torch.tensor([p]), 6, 50.0) * pf.rotate_pairs(y, torch.tensor([r]), 6, 50.0)).sum())
    assert abs(dot(10, 3) - dot(107, 100)) < 1e-9 and abs(dot(0, 0) - float((x * y).sum())) < 1e-12
    assert torch.equal(pf.rotate_pairs(x, torch.tensor([5]), 6, 50.0)[..., 6:], x[..., 6:])


def test_filters_and_the_delta_rule_carry_over_a_cut():
    g = torch.Generator().manual_seed(3)
    t, c, taps = 23, 5, 4
    x, w = torch.randn(t, c, generator=g, dtype=torch.float64), torch.randn(c, taps, generator=g, dtype=torch.float64)
    whole, _ = pf.short_conv(x, w)
    assert float((whole[0] - x[0] * w[:, -1]).abs().max()) < 1e-12       # the last column meets the current token
    assert float((whole[2] - (x[0] * w[:, 1] + x[1] * w[:, 2] + x[2] * w[:, 3])).abs().max()) < 1e-12
    a, kept = pf.short_conv(x[:2], w)
    b, _ = pf.short_conv(x[2:], w, kept)
    assert float((torch.cat([a, b]) - whole).abs().max()) < 1e-12
    heads, kd, vd = 2, 4, 3
    q, k = torch.randn(t, heads, kd, generator=g, dtype=torch.float64), torch.randn(t, heads, kd, generator=g, dtype=torch.float64)
    v = torch.randn(t, heads, vd, generator=g, dtype=torch.float64)
    beta, dec = torch.rand(t, heads, generator=g, dtype=torch.float64), torch.rand(t, heads, generator=g, dtype=torch.float64)
    o, s = pf.delta_rule(q, k, v, beta, dec)
    # the first token writes beta k v^T into an empty state and reads it at once
    assert float((o[0, 0] - beta[0, 0] * v[0, 0] * float(k[0, 0] @ q[0, 0])).abs().max()) < 1e-12
    o1, s1 = pf.delta_rule(q[:9], k[:9], v[:9], beta[:9], dec[:9])
    o2, s2 = pf.delta_rule(q[9:], k[9:], v[9:], beta[9:], dec[9:], s1)
    assert float((torch.cat([o1, o2]) - o).abs().max()) < 1e-12 and float((s2 - s).abs().max()) < 1e-12
    # with beta = 1 and a unit key the state answers the key with the value just written
    kk = k[5, 0] / k[5, 0].norm()
    _, s3 = pf.delta_rule(q[:1, :1], kk.view(1, 1, kd), v[5:6, :1], torch.ones(1, 1, dtype=torch.float64), dec[:1, :1], s[:1])
    assert float((s3[0].T @ kk - v[5, 0]).abs().max()) < 1e-12


def test_router_keeps_the_scores_of_the_chosen():
    z = torch.tensor([[0.0, 2.0, 2.0, -1.0]], dtype=torch.float64)
    ids, w = pf.route_softmax(z, 2)
    assert ids.tolist() == [[1, 2]] and abs(float(w.sum()) - float(torch.softmax(z, -1)[0, 1:3].sum())) < 1e-12


def test_plain_model_prefill_does_not_depend_on_later_tokens():
    import tempfile
    from tiny_llm_b200.config import FiponexConfig
    from tiny_llm_b200.weights import write_random_model
    for cfg in (FIP_B, FIP_C):
        d = write_random_model(tempfile.mkdtemp(), FiponexConfig.from_dict(cfg), seed=1, dtype=torch.float32)
        c, w = pf.load_config(d), pf.load_weights(d)
        toks = torch.randint(0, cfg["vocab"], (50,), generator=torch.Generator().manual_seed(1)).tolist()
        whole = pf.forward(c, w, toks)
        assert float((pf.forward(c, w, toks[:31]) - whole[:31]).abs().max()) < 1e-9


def test_a_replaced_workspace_buffer_stays_allocated():
    """Layers of unequal widths ask for one name with growing sizes inside one step; launches noted before the
    growth point into the smaller buffer, which must not be given to anything else while a tape can be replayed."""
    from tiny_llm_b200.engine import Workspace
    ws = Workspace(torch.device("cpu"))
    small = ws.get("rows", (3, 8), torch.float32)
    small.fill_(7.0)
    zeroed = ws.get_zeroed("sums", (3, 4))
    large = ws.get("rows", (3, 32), torch.float32)
    more = ws.get_zeroed("sums", (5, 4))
    assert large.data_ptr() != small.data_ptr() and more.data_ptr() != zeroed.data_ptr()
    held = {b.data_ptr() for b in ws.buffers()}
    assert {small.data_ptr(), large.data_ptr(), zeroed.data_ptr(), more.data_ptr()} <= held
    assert float(small.min()) == 7.0 and float(more.abs().max()) == 0.0
    assert ws.get("rows", (3, 32), torch.float32).data_ptr() == large.data_ptr()      # no growth: the same address
    assert ws.get("rows", (2, 8), torch.float32).data_ptr() == large.data_ptr()
