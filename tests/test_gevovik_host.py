"""Gevovik on the host: configuration and its errors, tensor names, cache needs (a latent layer that reads another
layer's cache keeps none; the token before is a state of the model), the block that norms what a branch gives, and the
plain implementation against closed forms."""
import copy

import pytest
import torch

import plain_gevovik as pg
from gevovik_util import GEV_A, GEV_B, GEV_C, GEV_D


def test_configuration_round_trip_and_spec():
    from tiny_llm_b200.config import GevovikConfig, config_from_dict
    for cfg in (GEV_A, GEV_B, GEV_C, GEV_D):
        c = config_from_dict(cfg)
        assert isinstance(c, GevovikConfig) and config_from_dict(c.to_dict()) == c
        spec = c.model_spec()
        assert spec.vocab_size == cfg["vocab"] and spec.hidden_size == cfg["width"] and len(spec.layers) == len(cfg["layers"])
        assert spec.embedding_scale == cfg["embedding"]["scale"]
        assert (spec.after_embedding is None) == ("bigram" not in cfg["embedding"])
        for layer, src, call in zip(spec.layers, cfg["layers"], spec.order):
            assert layer.block == "branch_norm" and layer.norm1.params["scalar"] and (layer.ffn is None) == (src["mlp"] is None)
            assert call.reads_cache_of == src["mixer"].get("kv_from")
            kind = {"mamba2": "mamba2", "latent_attention": "latent_attention", "parallel": "side_by_side"}[src["type"]]
            assert layer.mixer.kind == kind
    left = config_from_dict(GEV_A).model_spec().layers[0].mixer.params["branches"][0][1].params
    assert left["window"] == 20 and left["rot_scaling"]["factor"] == 2.0 and left["gate"] == "head" and left["talk"]
    assert config_from_dict(GEV_B).model_spec().layers[3].mixer.params["branches"][0][1].params["window"] is None


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][2]["mixer"].update(norm_groups=3), "norm_groups"),
    (lambda c: c["layers"][2]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "keeps no latents"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=16), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "unknown kind"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors_name_the_key(edit, word):
    from tiny_llm_b200.config import ConfigError, config_from_dict
    cfg = copy.deepcopy(GEV_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(cfg)


def test_tensor_names_and_cache_needs():
    from tiny_llm_b200.cache import CacheManager, KVNeed, StateNeed
    from tiny_llm_b200.config import config_from_dict
    from tiny_llm_b200.parts import DecoderModel
    model = DecoderModel(config_from_dict(GEV_A).model_spec())
    names = model.weight_specs()
    for n in ("embed", "bigram", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.left.q.norm", "l0.mix.left.talk",
              "l0.mix.left.temp", "l0.mix.left.g", "l0.mix.right.a1", "l0.mix.right.a2", "l0.mix.right.g2", "l0.mix.right.q.conv",
              "l0.mix.right.dt_bias", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.sink", "l2.mix.in", "l2.mix.conv.b", "l2.mix.D",
              "l3.mix.uk", "l3.mix.sink", "l0.mlp.up", "l0.mlp.down"):
        assert n in names, n
    for n in ("l3.mix.dkv", "l3.mix.dkv.norm", "l2.norm2", "l2.mlp.up", "l1.mix.g", "l0.mix.left.sink", "l0.mix.right.a"):
        assert n not in names, n
    assert names["final.norm"].shape == () and names["l0.norm1"].shape == () and names["bigram"].shape == (98, 64)
    assert names["l0.mix.left.g"].shape == (4, 64) and names["l0.mix.right.dt_bias"].shape == (4 * 16,)
    assert names["l2.mix.in"].shape == (2 * 64 + 2 * 2 * 16 + 4, 64) and names["l2.mix.norm"].shape == (64,)
    needs = model.cache_needs()
    assert len(needs) == 5 and needs[3] is None and needs[4] == StateNeed((1,), torch.int32)
    assert needs[0][0] == KVNeed(2, 16, 20, value_dim=32) and needs[0][1].shape == (4, 8, 16) and needs[0][2].shape == (3, 2 * 32 + 32)
    assert needs[1] == KVNeed(1, 32 + 16, None, value_dim=32)
    assert needs[2][0].shape == (4, 16, 16) and needs[2][1].shape == (3, 64 + 64)
    cache = CacheManager(needs, 128, 16, 2)
    assert len(cache.groups) == 2 and cache.refs[3].group is None and cache.refs[4].state is not None
    assert model.graph_safe
    # recurrent layers only: no page pool at all, and still a slot for the token before
    only = CacheManager(DecoderModel(config_from_dict(GEV_C).model_spec()).cache_needs(), 64, 8, 4)
    assert only.groups == [] and len(only.slots.needs) == 7
    # a model without bigram rows keeps nothing besides its layers' states
    assert len(DecoderModel(config_from_dict(GEV_B).model_spec()).cache_needs()) == 5


def test_pages_behind_the_window_go_back_and_the_shared_cache_keeps_its_own():
    from tiny_llm_b200.cache import CacheManager
    from tiny_llm_b200.config import config_from_dict
    from tiny_llm_b200.parts import DecoderModel
    cache = CacheManager(DecoderModel(config_from_dict(GEV_A).model_spec()).cache_needs(), 256, 16, 2)
    cache.add_request("a")
    assert cache.reserve("a", 100)
    cache.commit("a", 100)
    by_window = {g.need.window: g for g in cache.groups}
    assert by_window[None].pool.num_used == 7 and by_window[20].pool.num_used == 2
    cache.free_request("a")
    cache.check()
    assert all(g.pool.num_used == 0 for g in cache.groups)


def test_plain_pieces_against_closed_forms():
    g = torch.Generator().manual_seed(0)
    # bigram rows: the first token takes the row behind the buckets; the others depend on the pair alone
    assert pg.bigram_rows([5, 7, 7, 5], 11, 3, 2) == [11, (15 + 14) % 11, (21 + 14) % 11, (21 + 10) % 11]
    assert pg.bigram_rows([9], 4, 1, 1) == [4]
    # one number for all coordinates
    x = torch.randn(3, 10, generator=g, dtype=torch.float64)
    assert torch.allclose(pg.scalar_norm(x, 2.0, 0.0).pow(2).mean(-1), torch.full((3,), 4.0, dtype=torch.float64))
    # a rotation keeps lengths (times the magnitude) and scores depend on the distance alone, in both layouts
    f, mag = pg.rotation_frequencies(8, 100.0, {"factor": 4.0, "original": 16, "fast": 2.0, "slow": 0.5})
    q, k = torch.randn(1, 1, 12, generator=g, dtype=torch.float64), torch.randn(1, 1, 12, generator=g, dtype=torch.float64)
    for layout in ("halves", "pairs"):
        a = pg.rotate(q, torch.tensor([40]), f, mag, 8, layout)
        assert torch.allclose(a[..., :8].norm(), q[..., :8].norm() * mag) and torch.equal(a[..., 8:], q[..., 8:])
        s1 = (pg.rotate(q, torch.tensor([40]), f, mag, 8, layout) * pg.rotate(k, torch.tensor([33]), f, mag, 8, layout)).sum()
        s2 = (pg.rotate(q, torch.tensor([107]), f, mag, 8, layout) * pg.rotate(k, torch.tensor([100]), f, mag, 8, layout)).sum()
        assert torch.allclose(s1, s2)
    plain, one = pg.rotation_frequencies(8, 100.0)
    assert one == 1.0 and float(f[0]) == float(plain[0]) and float(f[-1]) == pytest.approx(float(plain[-1]) / 4.0)
    # a window of n keys: the token itself and n - 1 before it; a sink alone halves a lone key's weight at score 0
    v = torch.eye(6, dtype=torch.float64)[None]
    o = pg.masked_softmax_attention(torch.zeros(1, 6, 6, dtype=torch.float64), v, window=3)
    assert torch.allclose(o[5, 0], torch.tensor([0, 0, 0, 1 / 3, 1 / 3, 1 / 3], dtype=torch.float64))
    assert torch.allclose(o[1, 0], torch.tensor([0.5, 0.5, 0, 0, 0, 0], dtype=torch.float64))
    o = pg.masked_softmax_attention(torch.zeros(1, 6, 6, dtype=torch.float64), v, sink=torch.zeros(1))
    assert float(o[0, 0, 0]) == pytest.approx(0.5)
    # filters: zeros before the start, the last column at the current token
    y = pg.short_conv(torch.tensor([[1.0], [2.0], [3.0]]), torch.tensor([[10.0, 1.0]]), torch.tensor([0.5]))
    assert y.flatten().tolist() == [1.5, 12.5, 23.5]
    # recurrences carried over a cut: the delta rule with decays of 1 on a fresh key stores the value exactly
    k = torch.zeros(2, 1, 4, dtype=torch.float64)
    k[0, 0, 1] = k[1, 0, 2] = 1.0
    val = torch.randn(2, 1, 3, generator=g, dtype=torch.float64)
    o = pg.delta_rule_channel_decay(k, k, val, torch.ones(2, 1, 4, dtype=torch.float64), torch.ones(2, 1, dtype=torch.float64))
    assert torch.allclose(o, val)
    gk = torch.ones(2, 1, 4, dtype=torch.float64)
    gk[1, 0, 1] = 0.0      # the channel that holds the first value is wiped before the second token reads it
    q2 = torch.stack([k[0], k[0]])
    o = pg.delta_rule_channel_decay(q2, k, val, gk, torch.ones(2, 1, dtype=torch.float64))
    assert torch.allclose(o[1], torch.zeros(1, 3, dtype=torch.float64))
    # the state-space scan with decay 1 and unit steps sums b x^T
    x = torch.randn(3, 1, 2, generator=g, dtype=torch.float64)
    b = torch.ones(3, 1, 1, dtype=torch.float64)
    o = pg.state_space_scan(x, b, b, torch.ones(3, 1, dtype=torch.float64), torch.ones(3, 1, dtype=torch.float64))
    assert torch.allclose(o[:, 0], x[:, 0].cumsum(0))
