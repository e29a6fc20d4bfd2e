"""Gevovik through the engine against the plain implementation, in 32-bit and in bfloat16: whole prompts, the tail
decoded token by token, portions down to two tokens, mixed batches with pages and state slots used again, long
decoding across windows with pages given back, the residual stream layer by layer, and greedy generation through the
entry point and the command line.  Decoding carries the token before (the bigram rows), the recurrent states, the kept
filter inputs and, for a latent layer that reads another layer's cache, that layer's rows of the same step."""
import pytest
import torch

import plain_gevovik as pg
import replay_util as ru
from gevovik_util import GEV, compare, plain_logits, plain_model, tolerances, write_models

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [100, 64, 33, 47, 130, 17, 2, 51], "B": [97, 1, 40, 200, 33, 64, 13, 150], "C": [70, 90, 35, 49, 8],
           "D": [300, 131, 70, 260, 9]}


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    dirs = write_models(tmp_path_factory)
    out = {}
    for name, (cfg, page, seed) in GEV.items():
        reqs = ru.make_requests(cfg["vocab"], LENGTHS[name], seed + 20)
        out[name] = (dirs[name], cfg, page, reqs, {d: plain_logits(dirs[name], reqs, d) for d in DTYPES},
                     {d: tolerances(dirs[name], reqs, d) for d in DTYPES})
    return out


def runner_for(model_dir, dtype, page, max_tokens, max_requests=4, poison=True, per_step=1024, max_positions=None):
    from tiny_llm_b200.engine import load_model, make_runner
    _, model = load_model(model_dir, dtype, "cuda:0")
    runner = make_runner(model, dtype, "cuda:0", max_tokens=max_tokens, page_size=page, max_requests=max_requests,
                         max_tokens_per_step=per_step, max_positions=max_positions)
    if poison:   # a cache row that is read before it is written shows as NaN in the logits
        for g in runner.cache.groups:
            for t in g.tensors():
                t.fill_(float("nan"))
    return runner


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("how", ["whole", "tail", "portions", "mixed"])
def test_replay_in_process(cases, name, dtype, how):
    model_dir, cfg, page, reqs, ref, tol = cases[name]
    steps, prefix = {"whole": (ru.trace_whole(reqs), "w"), "tail": (ru.trace_tail(reqs), "t"),
                     "portions": (ru.trace_portions(reqs, 3), "p"), "mixed": (ru.trace_mixed(reqs, 4), "m")}[how]
    runner = runner_for(model_dir, dtype, page, ru.tokens_needed(steps, round_to=page))
    got = ru.run_trace_runner(runner, steps, cfg["vocab"])
    compare(got, ref[dtype], prefix, tol[dtype], f"gevovik {name} {how} {dtype}")
    assert all(g.pool.num_used == 0 for g in runner.cache.groups) and runner.cache.slots.num_free == 4
    if how == "mixed":   # more requests than state slots: slots were used again, and so were pages
        assert len(reqs) > 4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_trace_run_program(cases, name, dtype):
    """All four ways of cutting, through bin/trace_run as a user runs it, with the smallest pool and four slots."""
    model_dir, cfg, page, reqs, ref, tol = cases[name]
    some = dict(list(reqs.items())[:4])
    steps = (ru.trace_whole(some) + ru.trace_tail(some) + ru.trace_portions(some, 1) + ru.trace_mixed(reqs, 2))
    got = ru.run_trace_cli(model_dir, dtype, steps, cfg["vocab"])
    ref_some = {k: ref[dtype][k] for k in some}
    compare(got, ref_some, "w", tol[dtype], f"gevovik {name} whole (program) {dtype}")
    compare(got, ref_some, "t", tol[dtype], f"gevovik {name} tail (program) {dtype}")
    compare(got, ref_some, "p", tol[dtype], f"gevovik {name} portions (program) {dtype}")
    compare(got, ref[dtype], "m", tol[dtype], f"gevovik {name} mixed (program) {dtype}")


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_cuts_batches_and_pages_do_not_move_the_32_bit_logits(cases, name):
    """Whole, portions, and mixed batches with other page sizes and pools: the 32-bit path gives the same bits."""
    model_dir, cfg, page, reqs, ref, tol = cases[name]
    whole = ru.run_trace_runner(runner_for(model_dir, "float32", page, 4096), ru.trace_whole(reqs), cfg["vocab"])
    parts = ru.run_trace_runner(runner_for(model_dir, "float32", page, 4096), ru.trace_portions(reqs, 7), cfg["vocab"])
    steps = ru.trace_mixed(reqs, 9)
    mixed_a = ru.run_trace_runner(runner_for(model_dir, "float32", page, ru.tokens_needed(steps, page)), steps, cfg["vocab"])
    mixed_b = ru.run_trace_runner(runner_for(model_dir, "float32", 4 * page, 4096), steps, cfg["vocab"])
    for rid in reqs:
        assert torch.equal(whole["w" + rid], parts["p" + rid]), rid
        assert torch.equal(whole["w" + rid], mixed_a["m" + rid]), rid
        assert torch.equal(mixed_a["m" + rid], mixed_b["m" + rid]), rid


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_across_windows_with_graph_replays(cases, name, dtype):
    """A short prompt, then 290 tokens one by one: the windows pass many times, pages go back to the pool as a window
    leaves them, the token before, the recurrent states and the kept filter inputs are carried through every step, and
    the steps replay captured graphs."""
    model_dir, cfg, page, _, _, _ = cases[name]
    toks = ru.make_requests(cfg["vocab"], [300], 77)["r0"]
    ref = plain_logits(model_dir, {"r0": toks}, dtype)["r0"]
    runner = runner_for(model_dir, dtype, page, 304, max_positions=320)
    steps = ru.trace_tail({"r0": toks}, tail=290)
    got = ru.run_trace_runner(runner, steps, cfg["vocab"])
    compare(got, {"r0": ref}, "t", tolerances(model_dir, {"r0": toks}, dtype), f"gevovik long decoding {name} {dtype}")
    assert runner.graph_replays > 200


def test_pages_go_back_behind_the_window(cases):
    from tiny_llm_b200.engine import StepEntry
    model_dir, cfg, page, _, _, _ = cases["A"]   # a window of 20 tokens, pages of 16
    runner = runner_for(model_dir, "float32", page, 400, max_positions=400)
    runner.cache.add_request("x")
    toks = ru.make_requests(cfg["vocab"], [200], 3)["r0"]
    runner.step([StepEntry("x", toks, [0])])
    used = {g.need.window: g.pool.num_used for g in runner.cache.groups}
    assert used[None] == -(-200 // page) and used[20] <= -(-20 // page) + 1


def test_the_residual_stream_after_every_layer(cases):
    from tiny_llm_b200.engine import StepEntry
    for name in ("A", "B", "C", "D"):
        model_dir, cfg, page, _, _, _ = cases[name]
        toks = ru.make_requests(cfg["vocab"], [37], 5)["r0"]
        pc, pw, _ = plain_model(model_dir, "float32")
        streams = []
        pg.forward(pc, pw, toks, torch.float64, streams=streams)
        runner = runner_for(model_dir, "float32", page, 64)
        runner.use_graphs = runner.use_tapes = False
        seen = []
        runner.model.probe = lambda pos, x: seen.append(x.detach().clone().cpu())
        runner.cache.add_request("x")
        runner.step([StepEntry("x", toks, [0])])
        assert len(seen) == len(streams)
        for i, s in enumerate(seen):
            assert float((s.double() - streams[i]).abs().max()) <= 2e-5 * max(1.0, float(streams[i].abs().max())), (name, i)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(cases, name, dtype):
    from tiny_llm_b200 import Pipeline
    model_dir, cfg, page, _, _, _ = cases[name]
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 7, 30, 53, 12, 3)]
    pipe = Pipeline(model_dir, dtype=dtype, device=0, page_size=page, max_tokens=512, max_requests=4,
                    max_tokens_per_step=24, chunk=5)
    out = pipe.apply(prompts, max_new_tokens=40, do_sample=False, ignore_eos=True)
    assert [len(o) for o in out] == [40] * 6
    assert pipe.counters["chained"] > 0 and pipe.runner.graph_replays > 0
    pc, pw, quant = plain_model(model_dir, dtype)
    for p, o in zip(prompts, out):
        seq = list(p) + list(o)
        logits = pg.forward(pc, pw, seq, torch.float64)
        # a chosen token may trail the unrounded logits' best by what rounding moves two logits: in bfloat16, twice
        # (per logit) what rounding the activations does to the plain implementation on this very sequence
        slack = 2e-5 if dtype == "float32" else \
            4.0 * float((pg.forward(pc, pw, seq, torch.float64, quant=quant) - logits).abs().max())
        for i, tok in enumerate(o):
            row = logits[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= slack, (name, len(p), i)
    assert all(g_.pool.num_used == 0 for g_ in pipe.runner.cache.groups) and pipe.runner.cache.slots.num_free == 4
    if dtype == "float32":   # alone or in a batch: the same tokens
        assert pipe.apply([prompts[3]], max_new_tokens=40, do_sample=False, ignore_eos=True)[0] == out[3]


def test_the_command_line_generates_with_random_weights(tmp_path):
    import json
    import os
    import subprocess
    import sys
    cfg = GEV["B"][0]
    path = tmp_path / "config.json"
    path.write_text(json.dumps(cfg))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-m", "tiny_llm_b200", "--random_weights", f"--config={path}", "--seed=3",
                           "--max_new_tokens=5", "--nodo_sample", "--dtype=float32", "--page_size=4", "--max_tokens=256"],
                          input="5 6 7 8\n\n", text=True, capture_output=True, cwd=root, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    outs = [l for l in proc.stdout.splitlines() if l and l[0].isdigit()]
    assert len(outs) == 1 and len(outs[0].split()) == 5 and all(0 <= int(t) < cfg["vocab"] for t in outs[0].split())
    from tiny_llm_b200.config import GevovikConfig
    from tiny_llm_b200.weights import write_random_model
    d = write_random_model(str(tmp_path / "m"), GevovikConfig.from_dict(cfg), seed=3, dtype=torch.float32)
    seq = [5, 6, 7, 8]
    for tok in outs[0].split():
        row = pg.forward(pg.load_config(d), pg.load_weights(d), seq, torch.float64)[-1]
        assert float(row.max() - row[int(tok)]) <= 2e-5
        seq.append(int(tok))
