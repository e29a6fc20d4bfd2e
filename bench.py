#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, TinyLlama-1.1B layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

A step is one decode step of a batch of 8 requests at a context of 2,048 tokens (the last timed step
writes position 2047).  `value` is decoded tokens per second with the device clock around K steps
that are enqueued back to back; `e2e` is the same through the Python entry point with host tokens in
and out every step.  Every figure is the median of REPEATS timed regions of K steps each inside the
one run.  The line also carries a 2,048-token prefill, decoding at batch 1 and 64, the stated workload
of the model's benchmark (512-token prompts + 256 generated tokens through the entry point, admission and
prompts included), the same points at the Llama-2-7B and Llama-3-8B layer sizes (all 32 layers), the HBM
roofline of every decode point, and the clocks seen while timing.

`--design dunelix` measures another registered design instead (its own line, no record): prefill and decode of a
Dunelix model at the TinyLlama layer sizes beside the Llama decoder at equal sizes, and its kernels alone beside their
like kernels, each against its roofline (`--only decode` with it: the decode points alone).  `--design zozenex` does
the same for a Zozenex model (retention and gated linear attention, window attention with pooled blocks, routed
experts) beside the Dunelix model at equal width, layers and vocabulary, `--design gevovik` for a Gevovik model beside
the Fiponex model, `--design fiponex` for a Fiponex model (gated
delta rule, latent attention, attention with a sink, dense and routed gated feed-forwards) beside the Zozenex model."""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TINYLLAMA = dict(architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=22, hidden_size=2048,
                 num_attention_heads=32, num_key_value_heads=4, intermediate_size=5632, vocab_size=32000,
                 rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=2048, tie_word_embeddings=False,
                 hidden_act="silu", initializer_range=0.02, torch_dtype="bfloat16")
LLAMA2_7B = dict(TINYLLAMA, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=32,
                 intermediate_size=11008, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096)
LLAMA3_8B = dict(TINYLLAMA, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                 intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=8192)
OTHER_SHAPES = {"llama2_7b": (LLAMA2_7B, 3), "llama3_8b": (LLAMA3_8B, 4)}   # configuration, seed of its weights
CONTEXT = 2048
BATCH = 8
PAGE = 16
REPEATS = 5
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device=0):
        self.rows = []
        self.proc = None
        self.device = device

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.rows.append(parts)

    def stop(self):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(statistics.median(int(r[0]) for r in self.rows)), "sm_max_mhz": int(self.rows[0][1]),
                "reasons": reasons, "samples": len(self.rows)}


def build_model(layers, dtype, device, shape=TINYLLAMA, seed=2):
    import torch
    from tiny_llm_b200.config import LlamaConfig
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import load_state, random_state
    cfg = LlamaConfig.from_dict(dict(shape, num_hidden_layers=layers))
    model = DecoderModel(cfg.model_spec())
    specs = model.weight_specs()
    state = random_state(specs, seed, cfg.initializer_range, dtype, device=device)   # N(0, 0.02)
    model.load(load_state(specs, state, dtype, device))
    return cfg, model


def weight_bytes(model):
    """Bytes of every weight a decode step reads once: all matrices and norm vectors, not the
    embedding table (its rows are gathered)."""
    seen, total = set(), 0
    tensors = [model.lm_head, model.final_norm.weight]
    for b in model.blocks:
        tensors += [b.norm1.weight, b.norm2.weight, b.mixer.w_qkv, b.mixer.w_o, b.ffn.w_gate_up, b.ffn.w_down]
    for t in tensors:
        if t.data_ptr() not in seen:
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    return total


TRACE = os.environ.get("TLLM_TRACE") == "1"   # kernels built with timeline notes (a build for measurements)


def timeline_summary(records):
    """Per kind of launch (library, grid, block): how many, and the mean time in us from the moment the
    kernel before it had finished to the moment it had finished itself, inside the replayed graph."""
    kinds = {}
    for i, r in enumerate(records[:-1]):
        name = f"{r[6]} grid {r[2]}x{r[3]}x{r[4]} block {r[5]}"
        k = kinds.setdefault(name, [0, 0.0])
        k[0] += 1
        k[1] += (records[i + 1][1] - r[1]) / 1e3
    out = {n: {"launches": c, "mean_us": round(t / c, 2), "total_us": round(t, 1)} for n, (c, t) in kinds.items()}
    return dict(sorted(out.items(), key=lambda kv: -kv[1]["total_us"]))


def timed_decode(runner, batch, start_len, steps, warmup, sampler_out, repeats=1):
    """Prefills `batch` requests to start_len tokens, then runs warmup + repeats x steps decode steps enqueued
    back to back, each run of `steps` between two events; returns (median ms per step over the runs,
    kernels launched in one run, mean context of the timed steps)."""
    import torch
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import StepEntry
    g = torch.Generator().manual_seed(0)
    vocab = runner.model.spec.vocab_size
    rids = [f"d{batch}_{i}" for i in range(batch)]
    for rid in rids:
        assert runner.cache.add_request(rid) is not None
        toks = torch.randint(0, vocab, (start_len,), generator=g).tolist()
        for lo in range(0, start_len, 1024):
            runner.step([StepEntry(rid, toks[lo: lo + 1024], [])])
    feed = torch.randint(0, vocab, (warmup + repeats * steps, batch), generator=g).tolist()

    def one(i):
        logits = runner.step([StepEntry(rid, [feed[i][j]], [0]) for j, rid in enumerate(rids)])
        ops.argmax(logits, sampler_out[:batch])

    for i in range(warmup):
        one(i)
    times, launched = [], 0
    for rep in range(repeats):
        torch.cuda.synchronize()
        before = ops.launches
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(warmup + rep * steps, warmup + (rep + 1) * steps):
            if TRACE and rep == repeats - 1 and i == warmup + repeats * steps - 1:   # the last step alone, between two reads of the timeline notes
                torch.cuda.synchronize()
                ops.trace_dump()
            one(i)
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1) / steps)
        launched = ops.launches - before
    if TRACE:
        timed_decode.timeline = ops.trace_dump()
    for rid in rids:
        runner.cache.free_request(rid)
    mean_ctx = start_len + warmup + (repeats * steps + 1) / 2.0
    return statistics.median(times), launched, mean_ctx


def timed_prefill(runner, tokens, repeats=5):
    import torch
    from tiny_llm_b200.engine import StepEntry
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, runner.model.spec.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for i in range(repeats + 2):
        runner.cache.add_request("p")
        torch.cuda.synchronize()
        if TRACE and i == repeats + 1:   # the last step alone, between two reads of the timeline notes
            from tiny_llm_b200 import ops
            ops.trace_dump()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        runner.step([StepEntry("p", toks, [tokens - 1])])
        t1.record()
        torch.cuda.synchronize()
        if TRACE and i == repeats + 1:
            timed_prefill.timeline = ops.trace_dump()
        runner.cache.free_request("p")
        if i >= 2:
            times.append(t0.elapsed_time(t1))
    return statistics.median(times)


def timed_e2e(pipe, batch, context, steps, warmup, repeats=1):
    """The same decode through the Python entry point: host tokens in and out every step.  The
    requests are admitted over several steps (the prompt budget), so they get a margin of tokens
    that keeps all of them decoding side by side through warm-up and the timed steps; the last timed
    step still runs within `margin` tokens of `context`.  Returns the median over `repeats` runs of
    `steps` steps each of the wall time per step."""
    import torch
    from tiny_llm_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(3)
    vocab = pipe.model.spec.vocab_size
    margin = 2 * batch + 4
    new_tokens = repeats * steps + warmup + margin
    params = SamplingParams(max_new_tokens=new_tokens, do_sample=False, ignore_eos=True)
    for _ in range(batch):
        pipe.add_request(torch.randint(0, vocab, (context - new_tokens,), generator=g).tolist(), params)
    while any(r.remaining > 1 for r in pipe.scheduler.running) or pipe.scheduler.waiting:
        pipe.step()                                  # prompts in (untimed)
    for _ in range(warmup):
        pipe.step()
    times = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        assert len(pipe.scheduler.running) == batch
        t0 = time.perf_counter()
        for _ in range(steps):
            pipe.step()
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1e3 / steps)
        assert len(pipe.scheduler.running) == batch      # nobody ended inside the timed steps
    timed_e2e.h2d_bytes = pipe.runner.last_h2d_bytes     # of a timed step: tokens, positions, request and block tables
    while pipe.has_work():
        pipe.step()
    return statistics.median(times)


def timed_workload(pipe, batch, prompt_len=512, new_tokens=256, repeats=3):
    """The benchmark's stated workload through the entry point: `batch` requests of a 512-token random
    prompt each, 256 tokens generated greedily, from the first add_request to the last token on the
    host (admission, prompts in portions, decoding).  Returns generated tokens per second of wall time,
    median of `repeats` runs (after one untimed run)."""
    import torch
    g = torch.Generator().manual_seed(4)
    vocab = pipe.model.spec.vocab_size
    rates = []
    for rep in range(repeats + 1):
        prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in range(batch)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = pipe.apply(prompts, max_new_tokens=new_tokens, do_sample=False, ignore_eos=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        assert all(len(o) == new_tokens for o in out)
        if rep:
            rates.append(batch * new_tokens / dt)
    return statistics.median(rates)


def decode_bytes(model, runner, batch, mean_ctx, itemsize):
    """Bytes a decode step has to read: every weight once and the cache of the live requests."""
    kv_per_token = sum(g.bytes_per_token(itemsize) for g in runner.cache.groups)
    return weight_bytes(model) + batch * mean_ctx * kv_per_token


def prefill_flops(c, layers, t):
    """2 * T * matrix parameters + causal attention + LM head on one row."""
    per_layer = (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim +
                 c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    return 2.0 * t * per_layer * layers + 2.0 * t * t * c.num_attention_heads * c.head_dim * layers + \
        2.0 * c.hidden_size * c.vocab_size


def other_shape_points(name, shape, seed, dtype, device, pk, steps, out, points, fracs):
    """Decode at batch 16 and 64 and a 2,048-token prefill at another model's layer sizes, all of its layers."""
    import gc

    import torch
    from tiny_llm_b200.engine import make_runner
    cfg, model = build_model(shape["num_hidden_layers"], dtype, device, shape=shape, seed=seed)
    itemsize = 2 if dtype == torch.bfloat16 else 4
    runner = make_runner(model, dtype, device, max_tokens=64 * CONTEXT, page_size=PAGE, max_requests=64,
                         max_tokens_per_step=2048)
    s = min(steps, 16)
    for b in (16, 64):
        ms, _, ctx = timed_decode(runner, b, CONTEXT - (3 * s + 3), s, 3, out, repeats=3)
        points[f"{name}_decode_b{b}"] = round(b * 1e3 / ms, 1)
        fracs[f"{name}_decode_b{b}"] = round(decode_bytes(model, runner, b, ctx, itemsize) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    long_ctx = min(cfg.max_position_embeddings, 8192)
    if long_ctx > CONTEXT:   # a longer context where the model has the positions: 16 requests at 8,192 tokens
        ms, _, ctx = timed_decode(runner, 16, long_ctx - (3 * s + 3), s, 3, out, repeats=3)
        points[f"{name}_decode_b16_ctx{long_ctx}"] = round(16 * 1e3 / ms, 1)
        fracs[f"{name}_decode_b16_ctx{long_ctx}"] = round(decode_bytes(model, runner, 16, ctx, itemsize) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    ms = timed_prefill(runner, 2048, repeats=3)
    points[f"{name}_prefill_2048"] = round(2048 * 1e3 / ms, 1)
    if dtype == torch.bfloat16:
        fracs[f"{name}_prefill_2048"] = round(prefill_flops(cfg, cfg.num_hidden_layers, 2048) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
    del runner, model
    gc.collect()
    torch.cuda.empty_cache()


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def reference_arm(steps, warmup):
    """The reference arm: zscey/tiny-llm's own engine, unmodified (its parser, plan, runtime and CUDA kernels,
    compiled by baseline/build_reference.py and driven below the tokenizer by baseline/ref_driver.cpp as its
    Pipeline::apply drives it), at the same configuration: TinyLlama-1.1B layer sizes, 22 layers, batch 8,
    context 2,048, paged mode, greedy sampling on the host.  Its only dtype is float32.  pip cannot install
    the reference (no setup.py or pyproject.toml: a Bazel + Rust project), so the arm is built from its sources."""
    import tempfile
    exe = os.path.join(REF_DIR, "ref_driver")
    if not os.path.isfile(exe):
        try:
            res = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "build_reference.py")],
                                 capture_output=True, text=True, timeout=1500)
            why = (res.stderr.strip().splitlines() or res.stdout.strip().splitlines() or ["?"])[-1]
        except (OSError, subprocess.TimeoutExpired) as e:
            why = str(e)
        if not os.path.isfile(exe):
            print(json.dumps({"impl": "reference", "unavailable": f"the reference could not be built here: {why}"[:300]}))
            return 0
    cfg = dict(TINYLLAMA, torch_dtype="float32", eos_token_id=None, attention_bias=False, rope_scaling=None)
    pk = peaks()

    def run(mode, *extra):
        with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
            json.dump(cfg, f)
        try:
            res = subprocess.run([exe, mode, "--config", f.name] + [str(x) for x in extra], capture_output=True, text=True, timeout=900)
        finally:
            os.unlink(f.name)
        if res.returncode != 0:
            raise RuntimeError((res.stderr.strip().splitlines() or ["ref_driver failed"])[-1])
        return json.loads(res.stdout.strip().splitlines()[-1])

    try:
        sampler = ClockSampler().start()
        main_run = run("bench", "--batch", BATCH, "--context", CONTEXT, "--steps", steps, "--warmup", warmup, "--repeats", REPEATS)
        clocks = sampler.stop()
        s = min(steps, 8)
        points, notes = {}, {}
        for b in (1, 16, 64):
            try:
                r = run("bench", "--batch", b, "--context", CONTEXT, "--steps", s, "--warmup", 3, "--repeats", 3)
                points[f"decode_b{b}"] = round(b * 1e3 / r["ms_per_step_device"], 1)
            except RuntimeError as e:   # (at batch 64 the reference's own memory planner gives up: "Bad virtual block.")
                points[f"decode_b{b}"] = None
                notes[f"decode_b{b}"] = f"the reference does not run this batch: {e}"[:200]
        pre = run("prefill", "--tokens", 2048, "--repeats", 3)
    except (RuntimeError, OSError, subprocess.TimeoutExpired, ValueError) as e:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's engine did not run: {e}"[:300]}))
        return 0
    ms = main_run["ms_per_step_device"]
    weights = 4 * sum((TINYLLAMA["hidden_size"] * (TINYLLAMA["num_attention_heads"] + 2 * TINYLLAMA["num_key_value_heads"]) * 64 +
                       TINYLLAMA["hidden_size"] ** 2 + 3 * TINYLLAMA["hidden_size"] * TINYLLAMA["intermediate_size"]
                       for _ in range(TINYLLAMA["num_hidden_layers"]))) + 4 * TINYLLAMA["hidden_size"] * TINYLLAMA["vocab_size"]
    kv_per_token = 2 * TINYLLAMA["num_hidden_layers"] * TINYLLAMA["num_key_value_heads"] * 64 * 4
    mean_ctx = CONTEXT - (REPEATS * steps) / 2.0
    achieved = (weights + BATCH * mean_ctx * kv_per_token) / (ms * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8, context 2048 (TinyLlama-1.1B layer sizes)",
        "value": round(BATCH * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic", "impl": "reference",
        "config": {"model": "TinyLlama-1.1B shape, random weights", "global_batch": BATCH, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": 22, "layers_of_model": 22, "hidden_size": 2048, "heads": 32,
                   "kv_heads": 4, "head_dim": 64, "intermediate_size": 5632, "vocab_size": 32000, "page_size": 32,
                   "same_config": "sizes, batch and context as the other arm; float32 is the reference's only dtype, "
                                  "32 tokens its only page size", "peaks": pk["source"], "repeats": REPEATS,
                   "built_from": "unmodified tiny_llm/ sources, nvcc -arch=sm_100, driven by baseline/ref_driver.cpp"},
        "e2e": {"value": round(BATCH * 1e3 / main_run["ms_per_step_wall"], 1), "unit": "tokens/s",
                "ms_per_step": round(main_run["ms_per_step_wall"], 4), "h2d_bytes_per_step": main_run["h2d_bytes_per_step"],
                "d2h_bytes_per_step": main_run["d2h_bytes_per_step"]},
        "gpu_launches": None,
        "prefill": {"value": round(2048 * 1e3 / pre["ms"], 1), "tokens": 2048, "ms": round(pre["ms"], 3), "frac": None},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_note": notes, "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------- another design beside the flagship
# `--design dunelix`: prefill and decode of a Dunelix model (minGRU and chunked differential-attention layers, Dynamic
# Tanh) at layer sizes of the TinyLlama shape, beside the Llama decoder at equal width, feed-forward size, layers and
# vocabulary, and the new kernels alone beside their like kernels of the Llama path, each against its roofline.
DESIGN_LAYERS = 8


def dunelix_shape(layers=DESIGN_LAYERS, width=2048, ff=5632, vocab=32000, chunk=1024):
    att = {"type": "attention", "mixer": {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 128, "scale": 0.125, "diff": 0.4,
                                          "mask": {"size": chunk}, "rot": {"dims": 64, "base": 10000.0}},
           "mlp": {"kind": "dense", "ff": ff}}
    gru = {"type": "mingru", "mixer": {"width": width}, "mlp": {"kind": "dense", "ff": ff}}
    return {"architecture": "Dunelix", "vocab": vocab, "width": width, "residual_mult": 0.5, "norm": {"eps": 1e-6},
            "initializer_range": 0.02, "layers": [att if i % 4 == 3 else gru for i in range(layers)]}


def build_design(shape, dtype, device, seed=7):
    from tiny_llm_b200.config import config_from_dict
    from tiny_llm_b200.parts import DecoderModel
    from tiny_llm_b200.weights import load_state, random_state
    cfg = config_from_dict(shape)
    model = DecoderModel(cfg.model_spec())
    specs = model.weight_specs()
    model.load(load_state(specs, random_state(specs, seed, cfg.initializer_range, dtype, device=device), dtype, device))
    return cfg, model


def spec_weight_bytes(model, itemsize):
    """Bytes of every weight a decode step reads once (all but the embedding table, whose rows are gathered)."""
    from tiny_llm_b200.weights import COMPUTE
    total = 0
    for name, w in model.weight_specs().items():
        if name == model.spec.embed_name:
            continue
        n = 1
        for d in w.shape:
            n *= w.free_dim if d is None else d    # a rank that only the stored tensor fixes: what random weights use
        total += n * (itemsize if w.keep == COMPUTE else 4)
    return total


def design_decode_bytes(model, runner, batch, mean_ctx, itemsize):
    """Weights once, the keys and values each request can see (a chunked group: the part of its chunk behind it),
    and the recurrent states read and written."""
    total = spec_weight_bytes(model, itemsize)
    for g in runner.cache.groups:
        seen = mean_ctx if g.need.chunk is None else (mean_ctx % g.need.chunk or g.need.chunk)
        total += batch * seen * g.bytes_per_token(itemsize)
    total += 2 * batch * sum(4 * n.shape[0] for n in runner.cache.slots.needs)
    return total


def time_kernel(fn, flush, repeats=20):
    """Median microseconds of fn() with L2 flushed (a write of a buffer larger than L2) before every timed call."""
    import torch
    for _ in range(3):
        fn()
    times = []
    for _ in range(repeats):
        flush.zero_()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        fn()
        t1.record()
        torch.cuda.synchronize()
        times.append(t0.elapsed_time(t1) * 1e3)
    return statistics.median(times)


def design_kernels(dtype, device, pk, tokens=2048):
    """The new kernels alone at the sizes of one layer of the --design shape and `tokens` tokens of one prompt, and
    their like kernels of the Llama path at equal sizes: microseconds, achieved GB/s or TFLOP/s, share of the peak."""
    import types
    import torch
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    t, width, heads, kvh, kd, vd, chunk, page = tokens, 2048, 16, 4, 64, 128, 1024, PAGE
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    out = {}

    def mem(name, us, nbytes):
        out[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}

    def flop(name, us, flops):
        out[name] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}

    x = torch.randn(t, width, device=device)
    w, b, alpha = torch.ones(width, device=device), torch.zeros(width, device=device), torch.full((1,), 0.5, device=device)
    y = torch.empty(t, width, dtype=dtype, device=device)
    mem("dynamic_tanh", time_kernel(lambda: ops.dyt_norm(x, w, b, alpha, y), flush), t * width * 6)
    mem("rms_norm (like)", time_kernel(lambda: ops.rms_norm(x, w, 1e-5, y), flush), t * width * 6)

    zug = torch.randn(t, 3 * width, device=device).to(dtype)
    bias = torch.zeros(width, device=device)
    state = torch.zeros(4, width, device=device)
    batch = types.SimpleNamespace(cu_q=i32([0, t]), slots=i32([1]), num_requests=1, max_q_len=t)
    ws = Workspace(torch.device(device))
    yy = torch.empty(t, width, dtype=dtype, device=device)
    # segments read z and u twice: the algorithmic bytes are one read of [z|u|g] and one write of y
    mem("min_gru_scan", time_kernel(lambda: ops.min_gru_scan(zug, bias, bias, state, batch, yy, ws), flush), t * width * 8)
    gu = torch.randn(t, 2 * width, device=device).to(dtype)
    mem("silu_mul (like)", time_kernel(lambda: ops.silu_mul(gu, yy, 128), flush), t * width * 6)

    # one request of `t` tokens from position 0 in pages of its own
    pages = -(-t // page)
    table = i32([list(range(pages))])
    slots = i32(list(range(t)))
    pos = i32(list(range(t)))
    meta = types.SimpleNamespace(token_request=i32([0] * t), positions=pos, cu_q=i32([0, t]), q_start=i32([0]),
                                 num_requests=1, max_q_len=t, max_kv_len=t, num_leading_decodes=0)
    maps = 2
    qkv = torch.randn(t, (heads + kvh) * maps * kd + kvh * vd, device=device).to(dtype)
    kc = torch.zeros(pages, kvh * maps, page, kd, dtype=dtype, device=device)
    vc = torch.zeros(pages, kvh, page, vd, dtype=dtype, device=device)
    freq = torch.pow(torch.tensor(10000.0), -torch.arange(kd // 2, dtype=torch.float32) * 2 / kd).to(device)
    mem("rope_pairs_kv_write", time_kernel(lambda: ops.rope_pairs_kv_write(qkv, pos, freq, kd, heads * maps, kvh * maps, kvh, kd, vd,
                                                                          kc, vc, slots), flush),
        t * 2 * ((heads * maps * kd) * 2 + (kvh * maps * kd + kvh * vd) * 2))
    per_map = torch.empty(t, heads * maps * vd, dtype=torch.float32, device=device)
    # visible (query, key) pairs of a causal chunked mask
    pairs = sum(min(p % chunk, p) + 1 for p in range(t))
    att_flops = 2.0 * pairs * heads * maps * (kd + vd)
    flop("attention, two maps, chunk 1024", time_kernel(lambda: ops.paged_attention_maps(
        qkv, heads, kvh, maps, kd, vd, kc, vc, table, meta, per_map, 0.125, None, chunk), flush), att_flops)
    comb = torch.empty(t, heads * vd, dtype=dtype, device=device)
    lam = [torch.zeros(kd, device=device) for _ in range(4)]
    mem("diff_combine", time_kernel(lambda: ops.diff_combine(per_map.view(t, heads, maps, vd), *lam, 0.4, 1e-6, comb), flush),
        t * heads * vd * (8 + 2))
    # the like kernels of the Llama path at equal width: 32 heads of 64, 4 key/value heads
    lq = torch.randn(t, (32 + 8) * 64, device=device).to(dtype)
    lkv = torch.zeros(2, pages, 4, page, 64, dtype=dtype, device=device)
    cos = torch.ones(t, 32, device=device)
    sin = torch.zeros(t, 32, device=device)
    mem("rope_kv_write (like)", time_kernel(lambda: ops.rope_kv_write(lq, pos, cos, sin, 64, 32, 4, 64, lkv[0], lkv[1], slots), flush),
        t * 2 * (32 * 64 * 2 + 8 * 64 * 2))
    lo = torch.empty(t, 32 * 64, dtype=dtype, device=device)
    causal = sum(p + 1 for p in range(t))
    flop("attention (like: causal, 32 heads of 64)", time_kernel(lambda: ops.paged_attention(
        lq, 32, 4, 64, lkv[0], lkv[1], table, meta, lo, 0.125, None, ws), flush), 2.0 * causal * 32 * (64 + 64))
    return out


# `--design zozenex`: a Zozenex model (retention layers, every fourth layer window attention with pooled blocks beside
# gated linear attention, routed experts with a shared one) at the same width, layers and vocabulary, beside the Dunelix
# model above (the closest design the engine has: recurrent layers with an attention layer every fourth).
def zozenex_shape(layers=DESIGN_LAYERS, width=2048, vocab=32000, window=1024, pool=64):
    mlp = {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 32, "top": 4, "scale": 2.0}, "shared": {"ff": 1408}}
    ret = {"type": "retention", "mixer": {"heads": 16, "dim": 64, "vdim": 128,
                                          "decay": [1.0 - 2.0 ** -(5.0 + 0.25 * i) for i in range(16)]}, "mlp": mlp}
    par = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 128, "scale": 0.125, "softcap": 30.0,
                 "mask": {"size": window, "pool": pool}, "rot": {"dims": 64, "base": 10000.0}},
        "right": {"heads": 8, "dim": 64, "vdim": 128, "tau": 16.0, "rank": 16}}}
    return {"architecture": "Zozenex", "vocab": vocab, "width": width, "max_positions": CONTEXT, "norm": {"eps": 1e-6},
            "initializer_range": 0.02, "layers": [par if i % 4 == 3 else ret for i in range(layers)]}


def zozenex_decode_bytes(model, runner, batch, mean_ctx, itemsize):
    """What a decode step must move: the weights once (of the experts only those that the batch's tokens are expected
    to choose: E (1 - (1 - top / E)^batch) of E), the keys and values a request can see (its window and the block
    rows before it), and the recurrent states read and written."""
    total = 0
    for blk in model.blocks:
        f = blk.ffn
        expert = 0 if f is None else 2 * f.expert_size * f.hidden_size * itemsize
        chosen = 0.0 if f is None else f.num_experts * (1.0 - (1.0 - f.top / f.num_experts) ** batch)
        total += 0 if f is None else (chosen - f.num_experts) * expert     # spec_weight_bytes counts every expert
    total += spec_weight_bytes(model, itemsize)
    for g in runner.cache.groups:
        n = g.need
        if n.stride > 1:
            window = min(x.need.window for x in runner.cache.groups if x.need.window is not None)
            seen = max(0, mean_ctx - window)
        else:
            seen = mean_ctx if n.window is None else min(mean_ctx, n.window)
        total += batch * seen * g.bytes_per_token(itemsize)
    for n in runner.cache.slots.needs:
        numel = 1
        for d in n.shape:
            numel *= d
        total += 2 * batch * 4 * numel
    return int(total)


def zozenex_kernels(dtype, device, pk, tokens=2048):
    """The design's kernels alone at the sizes of one layer of the --design shape and `tokens` tokens of one prompt, and
    their like kernels of the Dunelix and Llama paths: microseconds, achieved GB/s or TFLOP/s, share of the peak."""
    import types
    import torch
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    t, width, heads, kvh, kd, vd, window, pool, page = tokens, 2048, 16, 4, 64, 128, 1024, 64, PAGE
    experts, top, ff = 32, 4, 1408
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    out = {}
    isz = 2 if dtype == torch.bfloat16 else 4

    def mem(name, us, nbytes):
        out[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}

    def flop(name, us, flops):
        out[name] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}

    ws = Workspace(torch.device(device))
    batch = types.SimpleNamespace(cu_q=i32([0, t]), slots=i32([1]), num_requests=1, max_q_len=t)
    # the recurrences: read q, k, v (and the gate's 32-bit rows), write 32-bit outputs
    for name, h, gated in (("linear_attention_scan (retention, 16 heads)", 16, False), ("linear_attention_scan (gated, 8 heads)", 8, True)):
        q, k = torch.randn(t, h * kd, device=device).to(dtype), torch.randn(t, h * kd, device=device).to(dtype)
        v = torch.randn(t, h * vd, device=device).to(dtype)
        state = torch.zeros(4, h, kd, vd, device=device)
        o = torch.empty(t, h * vd, device=device)
        kw = {"gate": torch.randn(t, h * kd, device=device), "gate_bias": torch.zeros(h * kd, device=device), "inv_tau": 1 / 16} \
            if gated else {"head_decay": torch.full((h,), 0.97, device=device)}
        mem(name, time_kernel(lambda: ops.linear_attention_scan(q, k, v, h, kd, vd, state, batch, o, 1.0, 0.125, workspace=ws, **kw), flush),
            t * h * ((2 * kd + vd) * isz + vd * 4 + (kd * 4 if gated else 0)))
        g = torch.randn(t, h * vd, device=device).to(dtype)
        y = torch.empty(t, h * vd, dtype=dtype, device=device)
        wn = torch.ones(vd, device=device)
        if not gated:
            mem("head_norm_gate", time_kernel(lambda: ops.head_norm_gate(o, wn, g, h, vd, 1e-6, y), flush), t * h * vd * (4 + 2 * isz))
    zug = torch.randn(t, 3 * width, device=device).to(dtype)
    bias = torch.zeros(width, device=device)
    st = torch.zeros(4, width, device=device)
    yy = torch.empty(t, width, dtype=dtype, device=device)
    mem("min_gru_scan (like)", time_kernel(lambda: ops.min_gru_scan(zug, bias, bias, st, batch, yy, ws), flush), t * width * 4 * isz)
    x = torch.randn(t, width, device=device)
    resid = torch.zeros(t, width, device=device)
    w1 = torch.ones(width, device=device)
    mem("rms_norm_add", time_kernel(lambda: ops.rms_norm_add(x, w1, 1e-6, 0.5, resid), flush), t * width * 16)
    mem("rms_norm (like)", time_kernel(lambda: ops.rms_norm(x, w1, 1e-6, yy), flush), t * width * (4 + isz))

    # one request of `t` tokens from position 0 in pages of its own
    pages = -(-t // page)
    table = i32([list(range(pages))])
    slots, pos = i32(list(range(t))), i32(list(range(t)))
    meta = types.SimpleNamespace(token_request=i32([0] * t), positions=pos, cu_q=i32([0, t]), q_start=i32([0]),
                                 num_requests=1, num_tokens=t, max_q_len=t, max_kv_len=t, num_leading_decodes=0)
    qkv = torch.randn(t, (heads + kvh) * kd + kvh * vd, device=device).to(dtype)
    kc = torch.zeros(pages, kvh, page, kd, dtype=dtype, device=device)
    vc = torch.zeros(pages, kvh, page, vd, dtype=dtype, device=device)
    pkc, pvc = torch.zeros_like(kc), torch.zeros_like(vc)
    fk = torch.pow(torch.tensor(10000.0), -torch.arange(kd // 2, dtype=torch.float32) * 2 / kd).to(device)
    fv = torch.pow(torch.tensor(10000.0), -torch.arange(vd // 2, dtype=torch.float32) * 2 / vd).to(device)
    mem("rope_halves_kv_write (values rotated)", time_kernel(lambda: ops.rope_halves_kv_write(
        qkv, pos, fk, kd, fv, heads, kvh, kvh, kd, vd, kc, vc, slots), flush), t * isz * (heads * kd * 2 + (kvh * kd + kvh * vd) * 2))
    pslots = i32([(p // pool) if (p + 1) % pool == 0 else -1 for p in range(t)])
    mem("pool_kv_blocks", time_kernel(lambda: ops.pool_kv_blocks(kc, vc, table, pkc, pvc, pslots, meta, pool), flush),
        t * kvh * (kd + vd) * isz * (1 + 1 / pool))
    att = torch.empty(t, heads * vd, dtype=dtype, device=device)
    hb = torch.zeros(heads, device=device)
    pairs = sum(min(p + 1, window) + max(0, (p - window - pool + 1) // pool + 1 if p - window - pool + 1 >= 0 else 0) for p in range(t))
    flop("window_pool_attention (window 1024, pool 64)", time_kernel(lambda: ops.window_pool_attention(
        qkv, heads, kvh, kd, vd, kc, vc, table, pkc, pvc, table, meta, att, 0.125, 30.0, hb, window, pool, fv), flush, repeats=5),
        2.0 * pairs * heads * (kd + vd))
    # like: the Dunelix attention (two maps, chunk 1024) and its rotation kernel
    maps = 2
    dq = torch.randn(t, (heads + kvh) * maps * kd + kvh * vd, device=device).to(dtype)
    dk = torch.zeros(pages, kvh * maps, page, kd, dtype=dtype, device=device)
    mem("rope_pairs_kv_write (like)", time_kernel(lambda: ops.rope_pairs_kv_write(dq, pos, fk, kd, heads * maps, kvh * maps, kvh, kd, vd,
                                                                                 dk, vc, slots), flush),
        t * isz * ((heads * maps * kd) * 2 + (kvh * maps * kd + kvh * vd) * 2))
    per_map = torch.empty(t, heads * maps * vd, dtype=torch.float32, device=device)
    dpairs = sum(min(p % 1024, p) + 1 for p in range(t))
    flop("attention, two maps, chunk 1024 (like)", time_kernel(lambda: ops.paged_attention_maps(
        dq, heads, kvh, maps, kd, vd, dk, vc, table, meta, per_map, 0.125, None, 1024), flush), 2.0 * dpairs * heads * maps * (kd + vd))

    # the experts: routing, grouping, the two grouped products, the combine; like: dense products of as many rows
    h_in = torch.randn(t, width, device=device).to(dtype)
    logits = torch.randn(t, experts + 1, device=device)
    corr = torch.zeros(experts, device=device)
    ids = torch.empty(t, top, dtype=torch.int32, device=device)
    wts = torch.empty(t, top, device=device)
    tile = ops.moe_tile_rows(t * top, experts, tensor_cores=dtype == torch.bfloat16)
    tiles = ops.moe_max_tiles(t * top, experts, tile)
    rows = torch.empty(tiles * tile, dtype=torch.int32, device=device)
    texp = torch.empty(tiles, dtype=torch.int32, device=device)

    def route():
        ops.moe_route(logits, experts, corr, 2.0, ids, wts)
        ops.moe_align(ids, experts, tile, rows, texp)
    mem("moe_route + moe_align", time_kernel(route, flush), t * (experts * 4 + top * 16))
    w_up = (torch.randn(experts, ff, width, device=device) * 0.02).to(dtype)
    w_down = (torch.randn(experts, width, ff, device=device) * 0.02).to(dtype)
    act = torch.empty(t * top, ff, dtype=dtype, device=device)
    yexp = torch.empty(t * top, width, device=device)
    flop("moe_linear up + gelu", time_kernel(lambda: ops.moe_linear(h_in, w_up, rows, texp, tile, act, rows_per_input=top, gelu=True), flush, repeats=5),
         2.0 * t * top * ff * width)
    flop("moe_linear down", time_kernel(lambda: ops.moe_linear(act, w_down, rows, texp, tile, yexp, rows_per_input=1), flush, repeats=5),
         2.0 * t * top * ff * width)
    if dtype == torch.bfloat16:
        # what prompt portions run: the grouped order made contiguous, both products on tcgen05 (tiles of 128 rows)
        t128 = ops.moe_max_tiles(t * top, experts, ops.MOE_TC_TILE)
        rows128 = torch.empty(t128 * 128, dtype=torch.int32, device=device)
        texp128 = torch.empty(t128, dtype=torch.int32, device=device)
        pos128 = torch.empty(t * top, dtype=torch.int32, device=device)
        ops.moe_align(ids, experts, 128, rows128, texp128, pos128)
        gin = torch.zeros(t128 * 128, width, dtype=dtype, device=device)
        gact = torch.zeros(t128 * 128, ff, dtype=dtype, device=device)
        gy = torch.zeros(t128 * 128, width, device=device)
        mem("moe_gather", time_kernel(lambda: ops.moe_gather(h_in, rows128, texp128, 128, gin, rows_per_input=top), flush),
            t * top * width * 2 * isz)
        flop("moe_linear_tc up + gelu (tcgen05)", time_kernel(lambda: ops.moe_linear_tc(gin, w_up, texp128, gact, gelu=True), flush),
             2.0 * t * top * ff * width)
        flop("moe_linear_tc down (tcgen05)", time_kernel(lambda: ops.moe_linear_tc(gact, w_down, texp128, gy), flush),
             2.0 * t * top * ff * width)
    dense_in = torch.randn(t * top, width, device=device).to(dtype)
    flop("linear of as many rows (like)", time_kernel(lambda: ops.linear(dense_in, w_up[0], act), flush), 2.0 * t * top * ff * width)
    shared = torch.randn(t, width, device=device)
    mem("moe_combine", time_kernel(lambda: ops.moe_combine(yexp, wts, shared, logits, experts, resid), flush),
        t * width * 4 * (top + 3))
    sact = torch.randn(t, ff, device=device).to(dtype)
    mem("gelu", time_kernel(lambda: ops.gelu(sact, sact), flush), t * ff * 2 * isz)
    gu = torch.randn(t, 2 * ff, device=device).to(dtype)
    mem("silu_mul (like)", time_kernel(lambda: ops.silu_mul(gu, sact, 128), flush), t * ff * 3 * isz)
    return out


# `--design fiponex`: a Fiponex model (gated delta rule layers, latent attention with a window, grouped-query attention with
# a sink, sandwich norms, dense gated feed-forwards and softmax-routed gated experts) at the same width, layers and
# vocabulary, beside the Zozenex model above (the closest design the engine has: matrix-state recurrences, a window
# attention every fourth layer, routed experts).
def fiponex_shape(layers=DESIGN_LAYERS, width=2048, vocab=32000, ff=5632, window=1024):
    moe = {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 32, "top": 4}}
    dense = {"kind": "dense", "ff": ff}
    delta = {"heads": 16, "kv_heads": 8, "dim": 128, "vdim": 128, "conv": 4}
    latent = {"heads": 16, "dim": 64, "rot_dim": 64, "vdim": 128, "kv_rank": 192, "scale": 128 ** -0.5,
              "mask": {"size": window}, "rot": {"dims": 64, "base": 10000.0}}
    att = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "q_temp": {"coef": 0.1, "every": 1024}}
    kinds = [("delta", delta, dense), ("delta", delta, moe), ("latent_attention", latent, moe), ("attention", att, dense)]
    return {"architecture": "Fiponex", "vocab": vocab, "width": width, "embedding": {"scale": width ** 0.5}, "norm": {"eps": 1e-6},
            "initializer_range": 0.02,
            "layers": [{"type": k, "mixer": m, "mlp": f} for k, m, f in (kinds[i % 4] for i in range(layers))]}


def fiponex_decode_bytes(model, runner, batch, mean_ctx, itemsize):
    """What a decode step must move: the weights once (of the experts only those that the batch's tokens are expected
    to choose: E (1 - (1 - top / E)^batch) of E), the cached rows a request can see (its window where the layer has
    one), and the recurrent states read and written."""
    total = spec_weight_bytes(model, itemsize)
    for blk in model.blocks:
        f = blk.ffn
        if f is None or not hasattr(f, "num_experts"):
            continue
        expert = (3 if f.glu is not None else 2) * f.expert_size * f.hidden_size * itemsize
        chosen = f.num_experts * (1.0 - (1.0 - f.top / f.num_experts) ** batch)
        total += (chosen - f.num_experts) * expert     # spec_weight_bytes counts every expert
    for g in runner.cache.groups:
        seen = mean_ctx if g.need.window is None else min(mean_ctx, g.need.window)
        total += batch * seen * g.bytes_per_token(itemsize)
    for n in runner.cache.slots.needs:
        numel = 1
        for d in n.shape:
            numel *= d
        total += 2 * batch * 4 * numel
    return int(total)

def fiponex_kernels(dtype, device, pk, tokens=2048):
    """The design's kernels alone at the sizes of one layer of the --design shape and `tokens` tokens of one prompt, and
    their like kernels of the Zozenex and Dunelix paths: microseconds, achieved GB/s or TFLOP/s, share of the peak."""
    import types
    import torch
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    t, width, page, window = tokens, 2048, PAGE, 1024
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    rnd = lambda *shape: torch.randn(*shape, device=device).to(dtype)
    out = {}
    isz = 2 if dtype == torch.bfloat16 else 4

    def mem(name, us, nbytes):
        out[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}

    def flop(name, us, flops):
        out[name] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}

    ws = Workspace(torch.device(device))
    pages = -(-t // page)
    table = i32([list(range(pages))])
    slots, pos = i32(list(range(t))), i32(list(range(t)))
    meta = types.SimpleNamespace(token_request=i32([0] * t), positions=pos, cu_q=i32([0, t]), q_start=i32([0]), slots=i32([1]),
                                 num_requests=1, num_tokens=t, max_q_len=t, max_kv_len=t, num_leading_decodes=0)

    # the gated delta rule: filters + unit norms + decays, the kept inputs, the recurrence, the per-head norm
    h, kvh, kd, vd, taps = 16, 8, 128, 128, 4
    ch = 2 * kvh * kd + h * vd
    proj = rnd(t, ch + h * vd + 2 * h)
    w_taps = torch.randn(ch, taps, device=device) * 0.5
    kept = torch.zeros(4, taps - 1, ch, device=device)
    q, k = torch.empty(t, kvh * kd, device=device), torch.empty(t, kvh * kd, device=device)
    v, gb = torch.empty(t, h * vd, device=device), torch.empty(t, h, 2, device=device)
    a_log, dt_bias = torch.zeros(h, device=device), torch.zeros(h, device=device)
    mem("delta_prepare (4 taps, unit norms, decays)", time_kernel(lambda: ops.delta_prepare(
        proj, w_taps, kept, meta, h, kvh, kd, vd, ch + h * vd, ch + h * vd + h, a_log, dt_bias, kd ** -0.5, 1e-6, q, k, v, gb), flush),
        t * ch * (isz + 4))
    mem("conv_state_update", time_kernel(lambda: ops.conv_state_update(proj, kept, meta, taps, ch), flush), (taps - 1) * ch * (isz + 4))
    state = torch.zeros(4, h, vd, kd, device=device)
    o = torch.empty(t, h * vd, device=device)
    scan_bytes = t * (2 * kvh * kd + 2 * h * vd + 2 * h) * 4
    scan_us = time_kernel(lambda: ops.delta_rule_scan(q, k, v, gb, state, meta, h, kvh, kd, vd, o), flush)
    mem("delta_rule_scan (16 heads, keys 128, values 128)", scan_us, scan_bytes)
    out["delta_rule_scan (16 heads, keys 128, values 128)"]["fp32_tflops"] = round(t * h * kd * vd * 8.0 / scan_us / 1e6, 2)
    state.zero_()
    lq, lk, lv = rnd(t, h * kd), rnd(t, h * kd), rnd(t, h * vd)
    lstate = torch.zeros(4, h, kd, vd, device=device)
    lkw = {"head_decay": torch.full((h,), 0.97, device=device)}
    like_us = time_kernel(lambda: ops.linear_attention_scan(lq, lk, lv, h, kd, vd, lstate, meta, o, 1.0, 0.125, workspace=ws, **lkw), flush)
    mem("linear_attention_scan (like; 16 heads, keys 128, values 128)", like_us, t * h * ((2 * kd + vd) * isz + vd * 4))
    out["linear_attention_scan (like; 16 heads, keys 128, values 128)"]["fp32_tflops"] = round(t * h * kd * vd * 4.0 / like_us / 1e6, 2)
    g = rnd(t, h * vd)
    y = torch.empty(t, h * vd, dtype=dtype, device=device)
    wn = torch.ones(vd, device=device)
    mem("head_norm_gate (shared with the like)", time_kernel(lambda: ops.head_norm_gate(o, wn, g, h, vd, 1e-6, y), flush), t * h * vd * (4 + 2 * isz))

    # grouped-query attention with a sink: biases + head norms + stretch + cache write, attention, the gate
    h, kvh, kd, vd = 16, 4, 128, 128
    width_in = (h + kvh) * kd + kvh * vd + h * vd
    qkv = rnd(t, width_in)
    kc = torch.zeros(pages, kvh, page, kd, dtype=dtype, device=device)
    vc = torch.zeros(pages, kvh, page, vd, dtype=dtype, device=device)
    bq, bk, bv = torch.zeros(h * kd, device=device), torch.zeros(kvh * kd, device=device), torch.zeros(kvh * vd, device=device)
    nq, nk = torch.ones(kd, device=device), torch.ones(kd, device=device)
    mem("qk_norm_kv_write (biases, head norms, stretch)", time_kernel(lambda: ops.qk_norm_kv_write(
        qkv, pos, h, kvh, kd, vd, kc, vc, slots, bq, bk, bv, nq, nk, eps=1e-6, stretch_coef=0.1, stretch_every=1024), flush),
        t * isz * (h * kd * 2 + (kvh * kd + kvh * vd) * 2))
    att = torch.empty(t, h * vd, dtype=torch.float32, device=device)
    sink = torch.zeros(h, device=device)
    pairs = t * (t + 1) // 2
    flop("attention with a sink (16 heads of 128, causal)", time_kernel(lambda: ops.paged_attention_maps(
        qkv, h, kvh, 1, kd, vd, kc, vc, table, meta, att, kd ** -0.5, None, None, sink=sink), flush, repeats=5), 2.0 * pairs * h * (kd + vd))
    gated = torch.empty(t, h * vd, dtype=dtype, device=device)
    off = (h + kvh) * kd + kvh * vd
    mem("sigmoid_gate (per value)", time_kernel(lambda: ops.sigmoid_gate(att, qkv[:, off:off + h * vd], h, vd, gated), flush), t * h * vd * (4 + 2 * isz))
    gu = rnd(t, 2 * h * vd)
    mem("silu_mul (like)", time_kernel(lambda: ops.silu_mul(gu, gated, 128), flush), t * h * vd * 3 * isz)

    # latent attention: norm + rotation + cache write, the queries into the latent's space, attention over one shared
    # row per token (key row 256 = latent 192 + rotated 64, value row 192), the values' projection per head
    h, nd, rd, lvd, rank = 16, 64, 64, 128, 192
    lkd = rank + rd
    lproj = rnd(t, -(-(h * (nd + rd) + lkd + h) // 8) * 8)
    lkc = torch.zeros(pages, 1, page, lkd, dtype=dtype, device=device)
    lvc = torch.zeros(pages, 1, page, rank, dtype=dtype, device=device)
    q_lat = torch.zeros(t, h, lkd, dtype=dtype, device=device)
    freq = torch.pow(torch.tensor(10000.0), -torch.arange(rd // 2, dtype=torch.float32) * 2 / rd).to(device)
    wl = torch.ones(rank, device=device)
    mem("latent_kv_write (norm, pair rotation)", time_kernel(lambda: ops.latent_kv_write(
        lproj, pos, h, nd, rd, rank, rd, freq, wl, 1e-6, q_lat, lkc, lvc, slots), flush), t * isz * (h * rd * 2 + lkd * 2 + rank))
    w_uk_t, w_uv = rnd(h, rank, nd), rnd(h, lvd, rank)
    flop("head_linear: latent query products (16 heads, 64 -> 192)", time_kernel(lambda: ops.head_linear(
        lproj[:, :h * (nd + rd)].view(t, h, nd + rd)[:, :, :nd], w_uk_t, q_lat[:, :, :rank]), flush), 2.0 * t * h * nd * rank)
    latt = torch.empty(t, h * rank, dtype=torch.float32, device=device)
    wpairs = sum(min(p + 1, window) for p in range(t))
    flop("latent attention (16 heads, key row 256, value row 192, window 1024)", time_kernel(lambda: ops.paged_attention_maps(
        q_lat.view(t, h * lkd), h, 1, 1, lkd, rank, lkc, lvc, table, meta, latt, 0.0884, window, None, sink=sink), flush, repeats=5),
        2.0 * wpairs * h * (lkd + rank))
    lg = torch.empty(t, h * rank, dtype=dtype, device=device)
    mem("sigmoid_gate (per head)", time_kernel(lambda: ops.sigmoid_gate(latt, lproj[:, h * (nd + rd) + lkd:h * (nd + rd) + lkd + h], h, rank, lg), flush),
        t * h * rank * (4 + isz))
    lout = torch.empty(t, h * lvd, dtype=dtype, device=device)

    flop("head_linear: latent value products (16 heads, 192 -> 128)", time_kernel(lambda: ops.head_linear(
        lg.view(t, h, rank), w_uv, lout.view(t, h, lvd)), flush), 2.0 * t * h * rank * lvd)
    # like: the Zozenex window attention with its rotation kernel, the Dunelix attention with two maps
    zh, zkv, zkd, zvd, pool = 16, 4, 64, 128, 64
    zq = rnd(t, (zh + zkv) * zkd + zkv * zvd)
    zk = torch.zeros(pages, zkv, page, zkd, dtype=dtype, device=device)
    zv = torch.zeros(pages, zkv, page, zvd, dtype=dtype, device=device)
    pkc, pvc = torch.zeros_like(zk), torch.zeros_like(zv)
    fk = torch.pow(torch.tensor(10000.0), -torch.arange(zkd // 2, dtype=torch.float32) * 2 / zkd).to(device)
    fv = torch.pow(torch.tensor(10000.0), -torch.arange(zvd // 2, dtype=torch.float32) * 2 / zvd).to(device)
    mem("rope_halves_kv_write (like)", time_kernel(lambda: ops.rope_halves_kv_write(zq, pos, fk, zkd, fv, zh, zkv, zkv, zkd, zvd, zk, zv, slots), flush),
        t * isz * (zh * zkd * 2 + (zkv * zkd + zkv * zvd) * 2))
    zo = torch.empty(t, zh * zvd, dtype=dtype, device=device)
    hb = torch.zeros(zh, device=device)
    zpairs = sum(min(p + 1, window) + max(0, (p - window - pool + 1) // pool + 1 if p - window - pool + 1 >= 0 else 0) for p in range(t))
    flop("window_pool_attention (like; window 1024, pool 64)", time_kernel(lambda: ops.window_pool_attention(
        zq, zh, zkv, zkd, zvd, zk, zv, table, pkc, pvc, table, meta, zo, 0.125, 30.0, hb, window, pool, fv), flush, repeats=5),
        2.0 * zpairs * zh * (zkd + zvd))
    maps = 2
    dq = rnd(t, (zh + zkv) * maps * zkd + zkv * zvd)
    dk = torch.zeros(pages, zkv * maps, page, zkd, dtype=dtype, device=device)
    per_map = torch.empty(t, zh * maps * zvd, dtype=torch.float32, device=device)
    dpairs = sum(min(p % 1024, p) + 1 for p in range(t))
    flop("attention, two maps, chunk 1024 (like)", time_kernel(lambda: ops.paged_attention_maps(
        dq, zh, zkv, maps, zkd, zvd, dk, zv, table, meta, per_map, 0.125, None, 1024), flush), 2.0 * dpairs * zh * maps * (zkd + zvd))

    # norms and the dense gate
    x = torch.randn(t, width, device=device)
    resid = torch.zeros(t, width, device=device)
    w1 = torch.ones(width, device=device)
    yy = torch.empty(t, width, dtype=dtype, device=device)
    mem("rms_norm_add (the norm behind a branch; shared with the like)", time_kernel(lambda: ops.rms_norm_add(x, w1, 1e-6, 1.0, resid), flush), t * width * 16)
    mem("rms_norm (shared with the like)", time_kernel(lambda: ops.rms_norm(x, w1, 1e-6, yy), flush), t * width * (4 + isz))
    ff = 5632
    du = rnd(t, 2 * ff)
    da = torch.empty(t, ff, dtype=dtype, device=device)
    mem("silu_mul with relu (dense gate; shared)", time_kernel(lambda: ops.silu_mul(du, da, 128, act="relu"), flush), t * ff * 3 * isz)

    # the experts: softmax routing and grouping, the gated grouped products on tcgen05, the combine
    experts, top, ff = 32, 4, 1408
    h_in = rnd(t, width)
    logits = torch.randn(t, experts, device=device)
    ids = torch.empty(t, top, dtype=torch.int32, device=device)
    wts = torch.empty(t, top, device=device)
    t128 = ops.moe_max_tiles(t * top, experts, ops.MOE_TC_TILE)
    rows128 = torch.empty(t128 * 128, dtype=torch.int32, device=device)
    texp128 = torch.empty(t128, dtype=torch.int32, device=device)
    pos128 = torch.empty(t * top, dtype=torch.int32, device=device)

    def route(softmax):
        ops.moe_route(logits, experts, None, 1.0, ids, wts, softmax=softmax)
        ops.moe_align(ids, experts, 128, rows128, texp128, pos128)
    mem("moe_route (sigmoid; like) + moe_align", time_kernel(lambda: route(False), flush), t * (experts * 4 + top * 16))
    mem("moe_route (softmax) + moe_align", time_kernel(lambda: route(True), flush), t * (experts * 4 + top * 16))
    if dtype == torch.bfloat16:
        w_up = (torch.randn(experts, 2 * ff, width, device=device) * 0.02).to(dtype)
        w_down = (torch.randn(experts, width, ff, device=device) * 0.02).to(dtype)
        gin = torch.zeros(t128 * 128, width, dtype=dtype, device=device)
        both = torch.zeros(t128 * 128, 2 * ff, device=device)
        gact = torch.zeros(t128 * 128, ff, dtype=dtype, device=device)
        gy = torch.zeros(t128 * 128, width, device=device)
        mem("moe_gather (shared with the like)", time_kernel(lambda: ops.moe_gather(h_in, rows128, texp128, 128, gin, rows_per_input=top), flush),
            t * top * width * 2 * isz)
        flop("moe_linear_tc gate and up (tcgen05, 32-bit sums out)", time_kernel(lambda: ops.moe_linear_tc(gin, w_up, texp128, both), flush),
             2.0 * t * top * 2 * ff * width)
        mem("silu_mul from 32-bit sums (gated experts)", time_kernel(lambda: ops.silu_mul(both, gact, ff, act="silu"), flush),
            t128 * 128 * ff * (8 + isz))
        flop("moe_linear_tc down (tcgen05; shared with the like)", time_kernel(lambda: ops.moe_linear_tc(gact, w_down, texp128, gy), flush),
             2.0 * t * top * ff * width)
        w_like = (torch.randn(experts, ff, width, device=device) * 0.02).to(dtype)
        flop("moe_linear_tc up + gelu (like)", time_kernel(lambda: ops.moe_linear_tc(gin, w_like, texp128, gact, gelu=True), flush),
             2.0 * t * top * ff * width)
    return out


# `--design gevovik`: a Gevovik model (latent attention with a sink over all earlier tokens, every second one of them
# reading the cache of the one before; a state-space mixer; a window attention with mixed scores beside a delta rule with
# decays per key channel; norms behind the branches; relu-squared feed-forwards; hashed bigram rows) at the same width,
# layers and vocabulary, beside the Fiponex model above (the closest design the engine has: latent attention, the
# delta rule, normed branches).
def gevovik_shape(layers=DESIGN_LAYERS, width=2048, vocab=32000, ff=5632, window=1024):
    dense = {"kind": "dense", "ff": ff}
    rot = {"dims": 64, "base": 10000.0}
    latent = {"heads": 16, "dim": 64, "rot_dim": 64, "vdim": 128, "kv_rank": 192, "scale": 128 ** -0.5, "rot": rot}
    mamba = {"heads": 32, "vdim": 128, "state": 128, "groups": 4, "norm_groups": 4, "conv": 4}
    par = {"left": {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": window},
                    "rot": {"dims": 128, "base": 10000.0, "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}},
           "right": {"heads": 16, "kv_heads": 8, "dim": 128, "vdim": 128, "conv": 4}, "left_scale": 0.5, "right_scale": 1.0}
    out = []
    for i in range(layers):
        if i % 4 == 0:
            out.append({"type": "latent_attention", "mixer": dict(latent), "mlp": dense})
        elif i % 4 == 1:
            out.append({"type": "mamba2", "mixer": mamba, "mlp": dense})
        elif i % 4 == 2:
            out.append({"type": "parallel", "mixer": par, "mlp": dense})
        else:
            out.append({"type": "latent_attention", "mixer": dict(latent, kv_from=i - 3), "mlp": dense})
    return {"architecture": "Gevovik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "initializer_range": 0.02,
            "embedding": {"scale": width ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 40009}}, "layers": out}


def gevovik_kernels(dtype, device, pk, tokens=2048):
    """The design's kernels alone at the sizes of one layer of the --design shape and `tokens` tokens of one prompt, and
    their like kernels of the Fiponex path: microseconds, achieved GB/s or TFLOP/s, share of the peak."""
    import types
    import torch
    from tiny_llm_b200 import ops
    from tiny_llm_b200.parts import stretched_frequencies
    t, width, page, window = tokens, 2048, PAGE, 1024
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    rnd = lambda *shape: torch.randn(*shape, device=device).to(dtype)
    out = {}
    isz = 2 if dtype == torch.bfloat16 else 4

    def mem(name, us, nbytes):
        out[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}

    def flop(name, us, flops):
        out[name] = {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)}

    pages = -(-t // page)
    table = i32([list(range(pages))])
    slots, pos = i32(list(range(t))), i32(list(range(t)))
    meta = types.SimpleNamespace(token_request=i32([0] * t), positions=pos, cu_q=i32([0, t]), q_start=i32([0]), slots=i32([1]),
                                 num_requests=1, num_tokens=t, max_q_len=t, max_kv_len=t, num_leading_decodes=0)

    # the left mixer: head norms + stretched rotation + cache write, the attention with mixed scores and a gate per head
    h, kvh, kd, vd = 16, 4, 128, 128
    qkv = rnd(t, (h + kvh) * kd + kvh * vd + h)
    kc = torch.zeros(pages, kvh, page, kd, dtype=dtype, device=device)
    vc = torch.zeros(pages, kvh, page, vd, dtype=dtype, device=device)
    nq, nk = torch.ones(kd, device=device), torch.ones(kd, device=device)
    freq, mag = stretched_frequencies(kd, 10000.0, {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0})
    freq = freq.to(device)
    mem("qk_norm_kv_write (head norms, stretched rotation in halves)", time_kernel(lambda: ops.qk_norm_kv_write(
        qkv, pos, h, kvh, kd, vd, kc, vc, slots, None, None, None, nq, nk, eps=1e-6, freq=freq, rot_mag=mag), flush),
        t * isz * (h * kd * 2 + (kvh * kd + kvh * vd) * 2))
    mem("qk_norm_kv_write (like: biases, head norms, stretch)", time_kernel(lambda: ops.qk_norm_kv_write(
        qkv, pos, h, kvh, kd, vd, kc, vc, slots, None, None, None, nq, nk, eps=1e-6, stretch_coef=0.1, stretch_every=1024), flush),
        t * isz * (h * kd * 2 + (kvh * kd + kvh * vd) * 2))
    mix = (torch.eye(h, device=device) + 0.1 * torch.randn(h, h, device=device)) * kd ** -0.5
    att = torch.empty(t, h * vd, dtype=dtype, device=device)
    off = (h + kvh) * kd + kvh * vd
    wpairs = sum(min(p + 1, window) for p in range(t))
    mix2 = (mix * 1.4426950408889634).contiguous()
    flop("attention_talk (16 heads of 128, 4 key/value heads, window 1024, mixed scores, gate per head)", time_kernel(
        lambda: ops.attention_talk(qkv, h, kvh, kd, vd, kc, vc, table, meta, mix, att, window=window, gate=qkv[:, off:off + h],
                                   mix_log2=mix2), flush, repeats=5), 2.0 * wpairs * h * (kd + vd + h))
    flop("attention_talk, the CUDA-core kernel of the 32-bit path on the same bfloat16 inputs", time_kernel(
        lambda: ops.attention_talk(qkv, h, kvh, kd, vd, kc, vc, table, meta, mix, att, window=window, gate=qkv[:, off:off + h]),
        flush, repeats=3), 2.0 * wpairs * h * (kd + vd + h))
    att32 = torch.empty(t, h * vd, dtype=torch.float32, device=device)
    sink = torch.zeros(h, device=device)
    flop("attention with a sink, window 1024 (like; tensor cores, scores not mixed)", time_kernel(lambda: ops.paged_attention_maps(
        qkv, h, kvh, 1, kd, vd, kc, vc, table, meta, att32, kd ** -0.5, window, None, sink=sink), flush, repeats=5),
        2.0 * wpairs * h * (kd + vd))

    # the right mixer: the delta rule with decays per key channel
    h, kvh, kd, vd, taps = 16, 8, 128, 128, 4
    ch = 2 * kvh * kd + h * vd
    proj = rnd(t, ch + 16 + h + 16)
    w_taps = torch.randn(ch, taps, device=device) * 0.5
    kept = torch.zeros(4, taps - 1, ch, device=device)
    q, k = torch.empty(t, kvh * kd, device=device), torch.empty(t, kvh * kd, device=device)
    v, gb = torch.empty(t, h * vd, device=device), torch.empty(t, h, 2, device=device)
    a_log, dt_h, dt_c = torch.zeros(h, device=device), torch.zeros(h, device=device), torch.zeros(h * kd, device=device)
    a_in, gk = torch.randn(t, h * kd, device=device), torch.empty(t, h * kd, device=device)
    mem("delta_prepare (decays per key channel)", time_kernel(lambda: ops.delta_prepare(
        proj, w_taps, kept, meta, h, kvh, kd, vd, ch + 16, ch + 16 + h, a_log, dt_c, kd ** -0.5, 1e-6, q, k, v, gb,
        mode="channel_decay", decay_in=a_in, gk=gk), flush), t * (ch * (isz + 4) + h * kd * 8))
    mem("delta_prepare (like: one decay per head)", time_kernel(lambda: ops.delta_prepare(
        proj, w_taps, kept, meta, h, kvh, kd, vd, ch + 16, ch + 16 + h, a_log, dt_h, kd ** -0.5, 1e-6, q, k, v, gb), flush),
        t * ch * (isz + 4))
    state = torch.zeros(4, h, vd, kd, device=device)
    o = torch.empty(t, h * vd, device=device)
    us = time_kernel(lambda: ops.delta_rule_scan(q, k, v, gb, state, meta, h, kvh, kd, vd, o, mode="channel_decay", gk=gk), flush)
    out["delta_rule_scan, decays per key channel (16 heads, 128 x 128)"] = {"us": round(us, 2), "fp32_tflops": round(t * h * kd * vd * 9.0 / us / 1e6, 2)}
    state.zero_()
    us = time_kernel(lambda: ops.delta_rule_scan(q, k, v, gb, state, meta, h, kvh, kd, vd, o), flush)
    out["delta_rule_scan, one decay per head (like; 16 heads, 128 x 128)"] = {"us": round(us, 2), "fp32_tflops": round(t * h * kd * vd * 8.0 / us / 1e6, 2)}
    state.zero_()
    g = rnd(t, h * vd)
    y = torch.empty(t, h * vd, dtype=dtype, device=device)
    wn = torch.ones(vd, device=device)
    mem("head_norm_gate with sigmoid (shared with the like)", time_kernel(lambda: ops.head_norm_gate(o, wn, g, h, vd, 1e-6, y, act="sigmoid"), flush),
        t * h * vd * (4 + 2 * isz))

    # the state-space mixer: 32 heads of 128 values, state 128, 4 groups
    h, groups, n, vd = 32, 4, 128, 128
    inner, bc = h * vd, groups * n
    ch = inner + 2 * bc
    proj = rnd(t, inner + ch + h)
    conv_in = proj[:, inner:]
    w_taps, b_taps = torch.randn(ch, taps, device=device) * 0.5, torch.zeros(ch, device=device)
    kept = torch.zeros(4, taps - 1, ch, device=device)
    q, k = torch.empty(t, bc, device=device), torch.empty(t, bc, device=device)
    v, gb = torch.empty(t, inner, device=device), torch.empty(t, h, 2, device=device)
    a_log, dt_h = torch.zeros(h, device=device), torch.zeros(h, device=device)
    mem("delta_prepare (state-space form: bias, step sizes)", time_kernel(lambda: ops.delta_prepare(
        conv_in, w_taps, kept, meta, h, groups, n, vd, ch, ch, a_log, dt_h, 1.0, 0.0, q, k, v, gb, mode="state_space",
        conv_bias=b_taps), flush), t * ch * (isz + 4))
    state = torch.zeros(4, h, vd, n, device=device)
    o = torch.empty(t, inner, device=device)
    us = time_kernel(lambda: ops.delta_rule_scan(q, k, v, gb, state, meta, h, groups, n, vd, o, mode="state_space"), flush)
    out["delta_rule_scan, state-space form (32 heads, state 128 x 128 values)"] = {"us": round(us, 2), "fp32_tflops": round(t * h * n * vd * 6.0 / us / 1e6, 2)}
    y = torch.empty(t, inner, dtype=dtype, device=device)
    wn = torch.ones(inner, device=device)
    skip = torch.ones(h, device=device)
    mem("gated_group_norm (skip, gate, 4 parts)", time_kernel(lambda: ops.gated_group_norm(
        o, proj[:, :inner], wn, 4, vd, 1e-6, y, skip_x=v, skip=skip), flush), t * inner * (8 + 2 * isz))

    # the stream: bigram rows, the copy a branch reads, the norm behind a branch, the weighted sum, relu squared
    x = torch.randn(t, width, device=device)
    resid = torch.zeros(t, width, device=device)
    tab = rnd(65522, width)
    toks = torch.randint(0, 32000, (t,), dtype=torch.int32, device=device)
    last = torch.zeros(4, 1, dtype=torch.int32, device=device)
    mem("bigram_add", time_kernel(lambda: ops.bigram_add(toks, tab, last, meta, resid, 1000003, 40009), flush), t * width * (isz + 8))
    emb = rnd(32000, width)
    mem("embedding (like)", time_kernel(lambda: ops.embedding(toks, emb, resid, scale=2.0), flush), t * width * (isz + 4))
    yy = torch.empty(t, width, dtype=dtype, device=device)
    mem("unary copy (the stream in the engine's dtype)", time_kernel(lambda: ops.unary(x, yy), flush), t * width * (4 + isz))
    w1 = torch.ones(width, device=device)
    mem("rms_norm (like)", time_kernel(lambda: ops.rms_norm(x, w1, 1e-6, yy), flush), t * width * (4 + isz))
    mem("rms_norm_add (the norm behind a branch; shared with the like)", time_kernel(lambda: ops.rms_norm_add(x, w1, 1e-6, 1.0, resid), flush), t * width * 16)
    mem("scaled_add (a side-by-side branch into the sum)", time_kernel(lambda: ops.scaled_add(x, 0.5, resid), flush), t * width * 16)
    ff = 5632
    sums = torch.randn(t, ff, device=device)
    act = torch.empty(t, ff, dtype=dtype, device=device)
    mem("unary relu squared from 32-bit sums", time_kernel(lambda: ops.unary(sums, act, "relu2"), flush), t * ff * (4 + isz))
    du = rnd(t, 2 * ff)
    mem("silu_mul with relu (like)", time_kernel(lambda: ops.silu_mul(du, act, 128, act="relu"), flush), t * ff * 3 * isz)
    return out


def design_run(args, dtype, device, pk):
    import gc
    import torch
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import make_runner
    itemsize = 2 if dtype == torch.bfloat16 else 4
    steps, warmup = min(max(1, args.steps), 32), max(3, min(args.warmup, 8))
    out = torch.zeros(64, dtype=torch.int32, device=device)
    sizes = {"dunelix": "width 2048, feed-forward 5632, vocabulary 32000; minGRU width 2048; attention 16 heads x 2 maps of 64, "
                        "4 key/value heads, values of 128, chunk 1024; every fourth layer attention; beside: Llama decoder, "
                        "32 heads of 64, 4 key/value heads, equal width, feed-forward, layers and vocabulary",
             "zozenex": "width 2048, vocabulary 32000; retention 16 heads, keys of 64, values of 128; every fourth layer window "
                        "attention (16 heads, 4 key/value heads, keys of 64, values of 128, window 1024, blocks of 64) beside gated "
                        "linear attention (8 heads, keys of 64, values of 128, rank 16); 32 experts of 1408, 4 chosen, a shared "
                        "expert of 1408; beside: the Dunelix model of --design dunelix at equal width, layers and vocabulary",
             "fiponex": "width 2048, vocabulary 32000; layers in turn: gated delta rule (16 heads, 8 query/key heads, keys and values "
                        "of 128, 4 taps) + dense gated feed-forward of 5632; the same + 32 gated experts of 1408, 4 chosen; latent "
                        "attention (16 heads, 64 plain + 64 rotated, values of 128, latent 192, window 1024) + experts; attention "
                        "with a sink (16 heads, 4 key/value heads, keys and values of 128, gate per value) + dense; beside: the "
                        "Zozenex model of --design zozenex at equal width, layers and vocabulary",
             "gevovik": "width 2048, vocabulary 32000, hashed bigram rows of 65521 buckets; layers in turn: latent attention with a "
                        "sink over all earlier tokens (16 heads, 64 plain + 64 rotated, values of 128, latent 192); state-space "
                        "mixer (32 heads of 128, state 128, 4 groups, 4 taps); window attention with mixed scores (16 heads, 4 "
                        "key/value heads, keys and values of 128, window 1024, stretched rotation, gate per head) beside a delta "
                        "rule with decays per key channel (16 heads, 8 query/key heads, keys and values of 128, 4 taps); latent "
                        "attention reading the first one's cache; every layer with a relu-squared feed-forward of 5632; beside: "
                        "the Fiponex model of --design fiponex at equal width, layers and vocabulary"}
    result = {"design": args.design, "dtype": args.dtype, "layers": DESIGN_LAYERS, "peaks": pk["source"],
              "sizes": sizes[args.design],
              "l2": "whole steps: weights larger than L2; kernels alone: L2 flushed before every timed call"}
    sampler = ClockSampler().start()
    labels = {"dunelix": ("dunelix", "llama"), "zozenex": ("zozenex", "dunelix"), "fiponex": ("fiponex", "zozenex"),
              "gevovik": ("gevovik", "fiponex")}[args.design]
    for label in labels[:1 if args.only == "decode" else 2]:
        if label == "dunelix":
            cfg, model = build_design(dunelix_shape(), dtype, device)
        elif label == "zozenex":
            cfg, model = build_design(zozenex_shape(), dtype, device)
        elif label == "fiponex":
            cfg, model = build_design(fiponex_shape(), dtype, device)
        elif label == "gevovik":
            cfg, model = build_design(gevovik_shape(), dtype, device)
        else:
            cfg, model = build_model(DESIGN_LAYERS, dtype, device)
        runner = make_runner(model, dtype, device, max_tokens=64 * CONTEXT, page_size=PAGE, max_requests=64,
                             max_tokens_per_step=2048, max_positions=CONTEXT)
        rec = {}
        for tt in (512, 2048) if args.only != "decode" else ():
            ms = timed_prefill(runner, tt, repeats=3)
            rec[f"prefill_{tt}"] = {"ms": round(ms, 3), "tokens_per_s": round(tt * 1e3 / ms, 1)}
        for bsz in (8, 64):
            ms, launched, ctx = timed_decode(runner, bsz, CONTEXT - (REPEATS * steps + warmup), steps, warmup, out, repeats=REPEATS)
            moved = design_decode_bytes(model, runner, bsz, ctx, itemsize) if label == "dunelix" else \
                zozenex_decode_bytes(model, runner, bsz, ctx, itemsize) if label == "zozenex" else \
                fiponex_decode_bytes(model, runner, bsz, ctx, itemsize) if label in ("fiponex", "gevovik") else \
                decode_bytes(model, runner, bsz, ctx, itemsize)
            rec[f"decode_b{bsz}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(bsz * 1e3 / ms, 1),
                                     "hbm_frac": round(moved / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4), "gpu_launches": launched}
        result[label] = rec
        del runner, model
        gc.collect()
        torch.cuda.empty_cache()
    result["clocks"] = sampler.stop()
    if dtype == torch.bfloat16 and args.only == "all":
        result["kernels"] = {"dunelix": design_kernels, "zozenex": zozenex_kernels, "fiponex": fiponex_kernels,
                             "gevovik": gevovik_kernels}[args.design](dtype, device, pk)
    ops.check_status()
    print(json.dumps(result))
    return 0


def main():
    global PAGE
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=TINYLLAMA["num_hidden_layers"],
                    help="fewer layers than the model has (layer sizes stay); both numbers are reported")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only (for profiler captures of a small case)")
    ap.add_argument("--batch", type=int, default=BATCH, help="requests of the decode step (default 8)")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens of the prompt step of --only prefill (default 2,048)")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="context the last timed step of --only decode reaches (default 2,048; at most the model's positions)")
    ap.add_argument("--page-size", type=int, default=PAGE, help="tokens per page of the cache")
    ap.add_argument("--shape", default="tinyllama", choices=["tinyllama"] + list(OTHER_SHAPES),
                    help="layer sizes for --only runs (profiler captures of the other models' kernels)")
    ap.add_argument("--design", default=None, choices=["dunelix", "zozenex", "fiponex", "gevovik"],
                    help="instead of the flagship run: this design's prefill and decode at real layer sizes beside the Llama "
                         "decoder at equal sizes, and its kernels beside their like kernels (one plain line, no record)")
    ap.add_argument("--quick", action="store_true",
                    help="leave out the workload points and the Llama-2-7B / Llama-3-8B layer sizes")
    args = ap.parse_args()
    PAGE = args.page_size
    if args.impl == "reference":
        return reference_arm(max(1, args.steps), max(3, args.warmup))
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    import torch
    from tiny_llm_b200 import Pipeline, ops
    from tiny_llm_b200.engine import make_runner, parse_dtype
    dtype = parse_dtype(args.dtype)
    device = "cuda:0"
    torch.cuda.set_device(0)
    pk = peaks()
    if args.design:
        return design_run(args, dtype, device, pk)
    if args.shape != "tinyllama" and args.only == "all":
        print("--shape goes with --only decode|prefill (the full run measures every shape)")
        return 2
    shape, seed = (TINYLLAMA, 2) if args.shape == "tinyllama" else OTHER_SHAPES[args.shape]
    cfg, model = build_model(min(args.layers, shape["num_hidden_layers"]), dtype, device, shape=shape, seed=seed)
    itemsize = 2 if dtype == torch.bfloat16 else 4
    start_len = CONTEXT - (REPEATS * steps + warmup)   # the last timed step writes position CONTEXT - 1
    if start_len < 64:
        print(f"--steps {steps} x {REPEATS} repeats + --warmup {warmup} do not fit a context of {CONTEXT}")
        return 2
    if args.only == "decode" and not 64 + steps + warmup <= args.context <= cfg.max_position_embeddings:
        print(f"--context {args.context}: the model has {cfg.max_position_embeddings} positions, and {steps} + {warmup} steps must fit")
        return 2
    pool_tokens = 64 * CONTEXT if args.only != "decode" else max(args.batch, 1) * (args.context + PAGE)
    runner = make_runner(model, dtype, device, max_tokens=pool_tokens, page_size=PAGE, max_requests=64,
                         max_tokens_per_step=2048)
    out = torch.zeros(64, dtype=torch.int32, device=device)

    if args.only != "all":
        # a small, single-purpose run for a profiler capture or a sweep: one plain line, no record
        if args.only == "decode":
            ms, launched, ctx = timed_decode(runner, args.batch, args.context - (steps + warmup), steps, warmup, out)
            moved = decode_bytes(model, runner, args.batch, ctx, itemsize)
            rec = {"only": "decode", "shape": args.shape, "batch": args.batch, "context": args.context,
                   "layers": cfg.num_hidden_layers, "ms_per_step": round(ms, 4),
                   "tokens_per_s": round(args.batch * 1e3 / ms, 1),
                   "hbm_frac": round(moved / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4), "gpu_launches": launched}
            if TRACE:
                rec["timeline"] = timeline_summary(timed_decode.timeline)
            print(json.dumps(rec))
        else:
            ops.attention_tc_timing(cfg.head_dim)   # (a build with cycle counters: start from zero)
            rec = {"only": "prefill", "shape": args.shape, "layers": cfg.num_hidden_layers, "tokens": args.tokens,
                   "ms": round(timed_prefill(runner, args.tokens, repeats=2), 3)}
            if TRACE:
                rec["timeline"] = timeline_summary(timed_prefill.timeline)
            cycles = ops.attention_tc_timing(cfg.head_dim)
            if cycles is not None:
                # cycles per key tile in the roles of the attention kernel's first CTA, which walks 2048 / 64 tiles
                tiles = (args.tokens // 64) * args.layers * 4
                rec["attention_cycles_per_tile"] = {n: round(v / tiles, 1) for n, v in cycles.items()}
            print(json.dumps(rec))
        return 0

    sampler = ClockSampler().start()
    ms, launched, mean_ctx = timed_decode(runner, BATCH, start_len, steps, warmup, out, repeats=REPEATS)
    clocks = sampler.stop()
    achieved = decode_bytes(model, runner, BATCH, mean_ctx, itemsize) / (ms * 1e-3) / 1e9

    points, fracs = {}, {}
    for b, key in ((1, "decode_b1"), (64, "decode_b64")):
        s = min(steps, 32)
        pms, _, ctx = timed_decode(runner, b, CONTEXT - (REPEATS * s + 3), s, 3, out, repeats=REPEATS)
        points[key] = round(b * 1e3 / pms, 1)
        fracs[key] = round(decode_bytes(model, runner, b, ctx, itemsize) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    prefill_ms = timed_prefill(runner, 2048)
    if not args.quick and dtype == torch.bfloat16:
        # shorter prompt steps: fewer tiles than SMs in every product
        for tt in (512, 1024):
            pms = timed_prefill(runner, tt, repeats=3)
            points[f"prefill_{tt}"] = round(tt * 1e3 / pms, 1)
            fracs[f"prefill_{tt}"] = round(prefill_flops(cfg, args.layers, tt) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)

    pipe = Pipeline.from_model(cfg, model, dtype=dtype, device=0, page_size=PAGE, max_tokens=BATCH * CONTEXT,
                               max_requests=BATCH, max_tokens_per_step=2048, chunk=1024)
    e2e_ms = timed_e2e(pipe, BATCH, CONTEXT, steps, warmup, repeats=REPEATS)
    h2d = timed_e2e.h2d_bytes
    del pipe

    # the stated workload of the model's benchmark: 512-token prompts + 256 generated tokens through the entry
    # point (generated tokens per second of wall time for the whole call, prompts and admission included)
    if not args.quick:
        for b in (1, 8, 64):
            wl = Pipeline.from_model(cfg, model, dtype=dtype, device=0, page_size=PAGE, max_tokens=b * 768 + 64,
                                     max_requests=b, max_tokens_per_step=2048, chunk=512)
            points[f"workload_512p_256g_b{b}"] = round(timed_workload(wl, b), 1)
            del wl

    c = cfg
    t = 2048
    flops = prefill_flops(c, args.layers, t)
    peak_flops = pk["bf16_tflops"] * 1e12 if dtype == torch.bfloat16 else None
    value = BATCH * 1e3 / ms
    if not args.quick:
        # the other shapes the benchmark names, all of their layers; this model's tensors go first
        del runner, model
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for name, (shape, seed) in OTHER_SHAPES.items():
            other_shape_points(name, shape, seed, dtype, device, pk, steps, out, points, fracs)
    line = {
        "metric": "decode tok/s at batch 8, context 2048 (TinyLlama-1.1B layer sizes)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else "fp32", "data": "synthetic", "impl": "ours",
        "config": {"model": "TinyLlama-1.1B shape, random weights seed 2", "global_batch": BATCH, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_of_model": TINYLLAMA["num_hidden_layers"],
                   "hidden_size": c.hidden_size, "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate_size": c.intermediate_size, "vocab_size": c.vocab_size,
                   "page_size": PAGE, "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": pk["source"], "repeats": REPEATS, "other_shapes": "llama2_7b and llama3_8b: 32 of 32 layers"},
        "e2e": {"value": round(BATCH * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * (BATCH + 1)},
        "gpu_launches": launched,
        # frac: of the burst peak of a library product timed alone; frac_of_sustained: of what the same product holds
        # back to back under the power cap, which is the state of the GPU inside a step of thousands of tokens
        "prefill": {"value": round(t * 1e3 / prefill_ms, 1), "tokens": t, "ms": round(prefill_ms, 3),
                    "frac": None if peak_flops is None else round(flops / (prefill_ms * 1e-3) / peak_flops, 4),
                    "frac_of_sustained": None if peak_flops is None else
                    round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "points_frac": fracs, "clocks": clocks,
        "libraries": sorted(os.path.basename(p) for p in ops.build.loaded_libraries().values()),
    }
    ops.check_status()   # no kernel of the timed runs gave up a bounded wait
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
