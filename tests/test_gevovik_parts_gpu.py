"""Each mechanism of Gevovik alone on the GPU against the plain implementation: the hashed bigram rows with the token
before carried in a state slot; the norm with one number and the block that norms what a branch gives; relu squared;
head norms with rotation in halves and in pairs, over a whole head and part of it, with stretched frequencies; the
attention whose heads' scores are mixed before the softmax (planted keys far back, at page borders, just inside and
just outside the window, on the first positions, in prompts and decoded alone, with a sink and a gate per head); the
delta rule with a decay per key channel and the state-space recurrence (from a state, for unequal requests, and the
same bits however a sequence is cut); the gated norm in parts; and the weighted sum of side-by-side branches."""
from types import SimpleNamespace

import pytest
import torch

import plain_gevovik as pg

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def close(got, ref, dtype, f32=2e-5, what=""):
    tol = f32 * max(1.0, float(ref.abs().max())) if dtype == torch.float32 else 2.0 ** -7 * float(ref.abs().max())
    worst = float((got.double().cpu() - ref.double()).abs().max())
    assert worst <= tol, (what, worst, tol)


def batch_of(q_lens, starts, slots=None):
    """The step's tables for requests that bring q_lens tokens behind `starts` earlier ones."""
    cu, req, pos = [0], [], []
    for i, (n, s) in enumerate(zip(q_lens, starts)):
        cu.append(cu[-1] + n)
        req += [i] * n
        pos += list(range(s, s + n))
    return SimpleNamespace(num_requests=len(q_lens), num_tokens=cu[-1], max_q_len=max(q_lens),
                           max_kv_len=max(s + n for s, n in zip(starts, q_lens)), cu_q=i32(cu), q_start=i32(starts),
                           token_request=i32(req), positions=i32(pos), slots=i32(slots or list(range(len(q_lens)))),
                           kv_len=i32([s + n for s, n in zip(starts, q_lens)]))


@pytest.mark.parametrize("dtype", DTYPES)
def test_bigram_rows_and_the_token_before(dtype):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(1)
    for buckets, mp, mc, width in [(13, 5, 3, 40), (1, 2, 9, 8), (1009, 1000003, 999983, 72)]:
        table = torch.randn(buckets + 1, width, generator=g).to(dtype)
        seqs = {0: torch.randint(0, 50000, (9,), generator=g).tolist(), 1: torch.randint(0, 50000, (4,), generator=g).tolist(),
                2: torch.randint(0, 50000, (1,), generator=g).tolist()}
        last = torch.full((4, 1), 12345, dtype=torch.int32, device=DEV)   # what a freed slot may still hold
        slot_of = {0: 2, 1: 0, 2: 3}
        done = {0: 0, 1: 0, 2: 0}
        # steps: portions beside single tokens, cut anywhere; a request is left out of a step and goes on later
        for step in ([(0, 3), (1, 1)], [(0, 1), (2, 1)], [(1, 3)], [(0, 5)]):
            q_lens = [n for _, n in step]
            b = batch_of(q_lens, [done[r] for r, _ in step], [slot_of[r] for r, _ in step])
            toks = [t for r, n in step for t in seqs[r][done[r]:done[r] + n]]
            x = torch.zeros(len(toks), width, device=DEV)
            ops.bigram_add(i32(toks), table.to(DEV), last, b, x, mp, mc)
            at = 0
            for r, n in step:
                rows = pg.bigram_rows(seqs[r], buckets, mp, mc)[done[r]:done[r] + n]
                assert torch.equal(x[at:at + n].cpu(), table[rows].float()), (buckets, r, done[r])
                at += n
                done[r] += n
                assert int(last[slot_of[r], 0]) == seqs[r][done[r] - 1]


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_with_one_number_behind_a_branch_and_relu_squared(dtype):
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    from tiny_llm_b200.parts import RMSNorm
    g = torch.Generator().manual_seed(2)
    for n, h, eps in [(5, 64, 1e-5), (33, 200, 1e-6), (3, 50, 1e-3)]:
        x = torch.randn(n, h, generator=g) * 3
        norm = RMSNorm(h, eps, weight_suffix="", scalar=True)
        assert norm.weight_specs("n")[0].shape == ()
        norm.load("n", {"n": torch.tensor(0.7, device=DEV)})
        ctx = SimpleNamespace(workspace=Workspace(torch.device(DEV)), dtype=dtype)
        ref = pg.scalar_norm(x.double(), 0.7, eps)
        resid = torch.randn(n, h, generator=g)
        branch, stream = x.to(DEV), resid.to(DEV)
        norm.add_into(ctx, branch, stream)
        close(stream, resid.double() + ref, torch.float32, what="normed branch added")
        assert float(branch.abs().max()) == 0.0     # the branch buffer is handed back zeroed
        out = torch.empty(n, h, dtype=dtype, device=DEV)
        ops.unary(x.to(DEV), out, "relu2")
        close(out, torch.relu(x.double()) ** 2, dtype, what="relu squared")
        ops.unary(x.to(DEV), out)
        assert torch.equal(out.cpu(), x.to(dtype))
        a, b = torch.randn(n, h, generator=g), torch.randn(n, h, generator=g)
        da, db = a.to(DEV), b.to(DEV)
        ops.scaled_add(da, 0.35, db)
        close(db, b.double() + 0.35 * a.double(), torch.float32, what="scaled add")
        assert float(da.abs().max()) == 0.0


def test_stretched_frequencies():
    from tiny_llm_b200.parts import stretched_frequencies
    for dims, base, sc in [(16, 100.0, None), (6, 30.0, (3.0, 8, 2.0, 0.5)), (32, 10000.0, (4.0, 64, 8.0, 1.0)),
                           (64, 300000.0, (16.0, 4096, 24.0, 1.5)), (8, 50.0, (2.0, 1000000, 1.0, 0.9))]:
        scaling = dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None
        f, mag = stretched_frequencies(dims, base, scaling)
        rf, rmag = pg.rotation_frequencies(dims, base, scaling)
        assert f.dtype == torch.float32 and float((f.double() - rf).abs().max() / rf.max()) < 1e-7 and abs(mag - rmag) < 1e-12
        if sc:   # the fastest pairs keep their frequency, the slowest are slowed by the factor
            plain, _ = pg.rotation_frequencies(dims, base)
            assert float(rf[0]) == float(plain[0]) or sc[1] > 100000
            assert mag == pytest.approx(0.1 * torch.log(torch.tensor(sc[0])).item() + 1.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_norms_rotation_and_cache_write(dtype):
    from tiny_llm_b200 import ops
    from tiny_llm_b200.parts import stretched_frequencies
    g = torch.Generator().manual_seed(5)
    cases = [(4, 2, 16, 24, 4, 16, "halves", (2.0, 16, 4.0, 1.0)), (6, 3, 10, 6, 8, 6, "halves", None),
             (3, 1, 40, 40, 4, 40, "pairs", (8.0, 64, 16.0, 2.0)), (2, 2, 48, 8, 16, 20, "pairs", None),
             (5, 5, 12, 12, 4, 0, "halves", None)]
    for nq, nkv, kd, vd, page, dims, layout, sc in cases:
        positions = [0, 1, 6, 7, 8, 15, 16, 700, 31999]
        t = len(positions)
        slots = [8, 9, 10, 20, 21, 1, 2, 3, 15]
        extra = 5      # columns behind q, k, v (a gate's) that the kernel must leave alone
        width = (nq + nkv) * kd + nkv * vd
        proj = torch.randn(t, width + extra, generator=g).to(dtype)
        wq, wk = torch.rand(kd, generator=g) + 0.5, torch.rand(kd, generator=g) + 0.5
        kc = torch.zeros(6, nkv, page, kd, dtype=dtype, device=DEV)
        vc = torch.zeros(6, nkv, page, vd, dtype=dtype, device=DEV)
        dev = proj.to(DEV)
        eps = 1e-5
        scaling = dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None
        freq, mag = stretched_frequencies(dims, 1000.0, scaling) if dims else (None, 1.0)
        ops.qk_norm_kv_write(dev, i32(positions), nq, nkv, kd, vd, kc, vc, i32(slots), None, None, None, wq.to(DEV),
                             wk.to(DEV), eps=eps, freq=None if freq is None else freq.to(DEV), rot_pairs=layout == "pairs",
                             rot_mag=mag)
        src = proj.double()
        q = pg.rms_unit(src[:, :nq * kd].view(t, nq, kd), eps) * wq.double()
        k = pg.rms_unit(src[:, nq * kd:(nq + nkv) * kd].view(t, nkv, kd), eps) * wk.double()
        if dims:
            rf, rmag = pg.rotation_frequencies(dims, 1000.0, scaling)
            q = pg.rotate(q, torch.tensor(positions), rf, rmag, dims, layout)
            k = pg.rotate(k, torch.tensor(positions), rf, rmag, dims, layout)
        v = src[:, (nq + nkv) * kd:width].view(t, nkv, vd)
        got = dev.cpu()
        # an angle of 31,999 radians is known to 2e-3 in 32-bit: the last positions get that much room
        close(got[:7, :nq * kd].view(7, nq, kd), q[:7], dtype, what=f"queries {layout} {dims}")
        close(got[7:, :nq * kd].view(2, nq, kd), q[7:], dtype, f32=4e-3, what=f"far queries {layout} {dims}")
        assert torch.equal(got[:, nq * kd:], proj[:, nq * kd:])     # nothing but the queries is rewritten in the row
        for i, s in enumerate(slots):
            close(kc[s // page, :, s % page].cpu(), k[i], dtype, f32=2e-5 if i < 7 else 4e-3, what="cached keys")
            close(vc[s // page, :, s % page].cpu(), v[i], dtype, what="cached values")


def talk_reference(q, k, v, mix, window, sink, gate, heads, kv_heads):
    """q [T, H, kd], k [T, G, kd], v [T, G, vd] of ONE sequence from position 0: the plain attention with mixed scores."""
    per = heads // kv_heads
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(per, dim=1))
    s = torch.einsum("hg,gij->hij", mix, s)
    o = pg.masked_softmax_attention(s, v.repeat_interleave(per, dim=1).transpose(0, 1), window=window, sink=sink)
    return o if gate is None else o * torch.sigmoid(gate)[:, :, None]


def paged(rows, page, n_pages, order, dtype):
    """rows [T, G, d] of one sequence into pages chosen by `order`; returns the cache and the sequence's block table."""
    t, g, d = rows.shape
    cache = torch.full((n_pages, g, page, d), float("nan"), dtype=dtype)
    table = order[: -(-t // page)]
    for i in range(t):
        cache[table[i // page], :, i % page] = rows[i].to(dtype)
    return cache, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(4, 2, 16, 32, 20, 16), (6, 3, 10, 6, 3, 4), (8, 1, 40, 24, 129, 32), (2, 2, 12, 12, None, 8),
                                   (5, 5, 8, 72, 64, 8), (16, 4, 20, 130, 33, 16), (24, 8, 8, 16, 17, 4),
                                   # sizes the tensor-core kernel takes in bfloat16
                                   (8, 2, 32, 16, 150, 32), (16, 4, 64, 48, 33, 16), (3, 1, 16, 16, None, 8), (12, 12, 128, 128, 100, 4)])
def test_mixed_scores_attention_with_planted_keys(dtype, sizes):
    """One sequence of 300 tokens, attended as a whole prompt, in portions, and with its last tokens decoded alone
    beside another request.  Planted: for chosen queries one key far back, at a page border, at the window's first
    position and right outside it gets a score that stands out in ONE head, which the mixing spreads to the others."""
    import math
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    heads, kvh, kd, vd, window, page = sizes
    ws = Workspace(torch.device(DEV))
    g = torch.Generator().manual_seed(heads * 100 + kd)
    t = 300
    q = torch.randn(t, heads, kd, generator=g) * 0.5
    k = torch.randn(t, kvh, kd, generator=g) * 0.5
    v = torch.randn(t, kvh, vd, generator=g)
    w = window or 10 ** 6
    for qi, back in [(299, w - 1), (298, w), (297, 1), (260, min(260, w - 1)), (250, min(250, w)), (5, 5), (1, 1), (0, 0),
                     (page * 9, page * 2), (page * 9 + 1, page * 2 + 1), (page * 9 - 1, page - 1), (280, 279 if window is None else 7)]:
        if qi - back < 0:
            continue
        h = qi % heads
        unit = k[qi - back, h // (heads // kvh)] / k[qi - back, h // (heads // kvh)].norm()
        q[qi, h] = unit * 12.0
    mix = torch.randn(heads, heads, generator=g) * 0.3 + torch.eye(heads)
    sink = torch.randn(heads, generator=g)
    gate = torch.randn(t, heads, generator=g)
    if dtype == torch.bfloat16:
        q, k, v, gate = (x.to(dtype).float() for x in (q, k, v, gate))
    n_pages = -(-t // page) + -(-40 // page) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    kc, table = paged(k, page, n_pages, order, dtype)
    vc, _ = paged(v, page, n_pages, order, dtype)
    # a second request of 40 tokens shares the pool
    other_pages = order[len(table): len(table) + -(-40 // page)]
    ko, vo, qo = torch.randn(40, kvh, kd, generator=g), torch.randn(40, kvh, vd, generator=g), torch.randn(40, heads, kd, generator=g)
    if dtype == torch.bfloat16:
        ko, vo, qo = (x.to(dtype).float() for x in (ko, vo, qo))
    for i in range(40):
        kc[other_pages[i // page], :, i % page] = ko[i].to(dtype)
        vc[other_pages[i // page], :, i % page] = vo[i].to(dtype)
    kc, vc = kc.to(DEV), vc.to(DEV)
    blocks = len(table) + 2
    for use_sink, use_gate in [(False, True), (True, False)]:
        ref = talk_reference(q.double(), k.double(), v.double(), mix.double(), window, sink.double() if use_sink else None,
                             gate.double() if use_gate else None, heads, kvh)
        ref_o = talk_reference(qo.double(), ko.double(), vo.double(), mix.double(), window, sink.double() if use_sink else None,
                               None, heads, kvh)

        def run(q_rows, gate_rows, q_lens, starts, tables):
            b = batch_of(q_lens, starts)
            bt = torch.full((len(q_lens), blocks), -1, dtype=torch.int32)
            for i, tb in enumerate(tables):
                bt[i, :len(tb)] = torch.tensor(tb)
            n = q_rows.shape[0]
            qd = torch.cat([q_rows.reshape(n, heads * kd), torch.zeros(n, 3)], dim=1).to(dtype).to(DEV)   # a row is longer than the queries
            out = torch.empty(n, heads * vd, dtype=torch.float32 if use_sink else dtype, device=DEV)
            ops.attention_talk(qd, heads, kvh, kd, vd, kc, vc, bt.to(DEV), b, mix.to(DEV), out, window=window,
                               sink=sink.to(DEV) if use_sink else None,
                               gate=gate_rows.to(dtype).to(DEV) if gate_rows is not None else None,
                               mix_log2=(mix.double() * math.log2(math.e)).float().to(DEV), workspace=ws)
            return out.view(n, heads, vd)

        def gates(rows):
            return rows if use_gate else None
        whole = run(q, gates(gate), [t], [0], [table])
        close(whole, ref, dtype, what=f"whole prompt {sizes}")
        # portions of 2, 7, 1 and more tokens of the long request beside a portion and then single tokens of the other
        at, at_o, got, got_o = 0, 0, [], []
        for n, n_o in [(2, 9), (7, 1), (1, 1), (150, 20), (33, 0), (100, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1), (1, 1)]:
            if n_o:
                out = run(torch.cat([qo[at_o:at_o + n_o], q[at:at + n]]),
                          torch.cat([torch.zeros(n_o, heads) + 50.0, gate[at:at + n]]) if use_gate else None,
                          [n_o, n], [at_o, at], [other_pages, table])
                got_o.append(out[:n_o])
                got.append(out[n_o:])
            else:
                got.append(run(q[at:at + n], gates(gate[at:at + n]), [n], [at], [table]))
            at, at_o = at + n, at_o + n_o
        assert at == t
        close(torch.cat(got), ref, dtype, what=f"portions and decoded tokens {sizes}")
        close(torch.cat(got_o), ref_o[:at_o], dtype, what=f"the other request {sizes}")
        if dtype == torch.float32:   # how the prompt was cut does not move a bit
            assert torch.equal(torch.cat(got), whole)


def recurrence_inputs(g, t, heads, kvh, kd, vd):
    q, k = torch.randn(t, kvh, kd, generator=g), torch.randn(t, kvh, kd, generator=g)
    q, k = q / q.norm(dim=-1, keepdim=True) * kd ** -0.5, k / k.norm(dim=-1, keepdim=True)
    return q, k, torch.randn(t, heads, vd, generator=g)


@pytest.mark.parametrize("sizes", [(4, 2, 16, 8), (2, 1, 6, 10), (3, 3, 33, 20), (8, 2, 48, 32), (2, 2, 128, 17), (1, 1, 100, 64),
                                   (2, 1, 200, 24), (1, 1, 256, 16)])
def test_delta_rule_with_a_decay_per_key_channel(sizes):
    from tiny_llm_b200 import ops
    heads, kvh, kd, vd = sizes
    g = torch.Generator().manual_seed(kd)
    lens = [37, 1, 90]
    outs, states = [], torch.zeros(5, heads, vd, kd, device=DEV)
    slots = [3, 0, 4]
    data = []
    for n in lens:
        q, k, v = recurrence_inputs(g, n, heads, kvh, kd, vd)
        gk = torch.rand(n, heads, kd, generator=g) * 0.5 + 0.5
        gk[:, :, 0] = 1.0
        gk[n // 2, 0] = 0.0          # a channel-wise reset in the middle
        beta = torch.rand(n, heads, generator=g)
        data.append((q, k, v, gk, beta))
    per = heads // kvh
    refs = [pg.delta_rule_channel_decay(q.double().repeat_interleave(per, 1), k.double().repeat_interleave(per, 1), v.double(),
                                        gk.double(), beta.double()) for q, k, v, gk, beta in data]

    def run(cuts, state):
        """cuts[i]: how many tokens request i brings per step (0: it sits the step out)."""
        got = [[] for _ in lens]
        done = [0] * len(lens)
        for step in zip(*cuts):
            live = [i for i, n in enumerate(step) if n]
            b = batch_of([step[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
            cat = lambda j: torch.cat([data[i][j][done[i]:done[i] + step[i]] for i in live])
            n = b.num_tokens
            gb = torch.stack([torch.ones(n, heads), cat(4)], dim=-1).contiguous()
            out = torch.empty(n, heads * vd, device=DEV)
            ops.delta_rule_scan(cat(0).reshape(n, -1).contiguous().to(DEV), cat(1).reshape(n, -1).contiguous().to(DEV),
                                cat(2).reshape(n, -1).contiguous().to(DEV), gb.to(DEV), state, b, heads, kvh, kd, vd, out,
                                mode="channel_decay", gk=cat(3).reshape(n, -1).contiguous().to(DEV))
            at = 0
            for i in live:
                got[i].append(out[at:at + step[i]].view(step[i], heads, vd).cpu())
                at += step[i]
                done[i] += step[i]
        return [torch.cat(x) for x in got]
    whole = run([[37], [1], [90]], states.clone())
    for got, ref in zip(whole, refs):
        close(got, ref, torch.float32, f32=1e-4, what=f"channel decay {sizes}")
    parts = run([[2, 30, 0, 5], [0, 0, 1, 0], [1, 1, 80, 8]], states.clone())
    for a, b in zip(whole, parts):
        assert torch.equal(a, b)     # the same operations on every state element however the sequence is cut


@pytest.mark.parametrize("sizes", [(4, 2, 16, 16), (6, 3, 10, 6), (5, 5, 12, 8), (2, 1, 7, 20), (8, 2, 64, 32), (16, 16, 32, 8)])
def test_state_space_recurrence_and_the_gated_norm_in_parts(sizes):
    from tiny_llm_b200 import ops
    heads, groups, n_state, vd = sizes
    g = torch.Generator().manual_seed(n_state + vd)
    t = 75
    x = torch.randn(t, heads, vd, generator=g)
    bmat, cmat = torch.randn(t, groups, n_state, generator=g), torch.randn(t, groups, n_state, generator=g)
    dt = torch.rand(t, heads, generator=g) * 2
    decay = torch.exp(-torch.rand(heads, generator=g) * dt)
    per = heads // groups
    ref = pg.state_space_scan(x.double(), bmat.double().repeat_interleave(per, 1), cmat.double().repeat_interleave(per, 1),
                              decay.double(), dt.double())
    state = torch.zeros(3, heads, vd, n_state, device=DEV)
    gb = torch.stack([decay, dt], dim=-1).contiguous().to(DEV)
    got = []
    at = 0
    for n in (1, 2, 40, 32):   # the sequence in portions, its state carried in slot 2
        b = batch_of([n], [at], [2])
        out = torch.empty(n, heads * vd, device=DEV)
        ops.delta_rule_scan(cmat[at:at + n].reshape(n, -1).contiguous().to(DEV), bmat[at:at + n].reshape(n, -1).contiguous().to(DEV),
                            x[at:at + n].reshape(n, -1).contiguous().to(DEV), gb[at:at + n].contiguous(), state, b, heads, groups,
                            n_state, vd, out, mode="state_space")
        got.append(out.cpu())
        at += n
    o = torch.cat(got)
    close(o.view(t, heads, vd), ref, torch.float32, f32=1e-4, what=f"state space {sizes}")
    skip = torch.randn(heads, generator=g)
    w = torch.rand(heads * vd, generator=g) + 0.5
    for dtype in DTYPES:
        for parts in [p for p in (1, 2, heads, heads * vd) if (heads * vd) % p == 0]:
            z = torch.randn(t, heads * vd + 3, generator=g).to(dtype)
            y = torch.empty(t, heads * vd, dtype=dtype, device=DEV)
            ops.gated_group_norm(o.to(DEV), z.to(DEV)[:, :heads * vd], w.to(DEV), parts, vd, 1e-5, y,
                                 skip_x=x.reshape(t, -1).contiguous().to(DEV), skip=skip.to(DEV))
            full = (o.double().view(t, heads, vd) + skip.double()[None, :, None] * x.double()).reshape(t, -1) * pg.silu(z[:, :heads * vd].double())
            want = (pg.rms_unit(full.view(t, parts, -1), 1e-5).reshape(t, -1) * w.double())
            close(y, want, dtype, what=f"gated norm in {parts} parts")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prepare_kernels_of_both_recurrences(dtype):
    """Filters from kept inputs (with and without a bias), SiLU, unit vectors or none, decays per channel and step sizes,
    for two requests of which one continues from a state."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(11)
    for heads, kvh, kd, vd, taps in [(4, 2, 16, 8, 4), (2, 1, 6, 10, 1), (3, 3, 8, 8, 3), (6, 2, 10, 6, 2)]:
        qk, vg = kvh * kd, heads * vd
        ch = 2 * qk + vg
        lens, starts = [9, 5], [0, 6]
        t = sum(lens)
        b = batch_of(lens, starts, [1, 0])
        hist = torch.randn(starts[1], ch + heads, generator=g).to(dtype).float()      # what request 1 saw before this step
        kept = torch.zeros(2, max(taps - 1, 1), ch, device=DEV)
        if taps > 1:
            kept[0, -min(taps - 1, starts[1]):] = hist[-min(taps - 1, starts[1]):, :ch].to(DEV)
        proj = torch.randn(t, ch + heads + 2, generator=g).to(dtype)
        w_taps = torch.randn(ch, taps, generator=g) * 0.5
        a_log, bias = torch.rand(heads, generator=g) - 1.0, torch.randn(ch, generator=g) * 0.2
        q, k = torch.empty(t, qk, device=DEV), torch.empty(t, qk, device=DEV)
        v, gb = torch.empty(t, vg, device=DEV), torch.empty(t, heads, 2, device=DEV)
        seqs = [proj[:9].float(), torch.cat([hist, proj[9:, :ch + heads].float()])]

        def conv(seq, bias_):
            return pg.silu(pg.short_conv(seq[:, :ch].double(), w_taps.double(), bias_))
        # the delta rule with decays per channel: channels [q | k | v], unit vectors, beta = sigmoid, g from rows of their own
        dt_bias = torch.randn(heads * kd, generator=g)
        a_in = torch.randn(t, heads * kd, generator=g)
        gk = torch.empty(t, heads * kd, device=DEV)
        ops.delta_prepare(proj.to(DEV), w_taps.to(DEV), kept, b, heads, kvh, kd, vd, ch, ch, a_log.to(DEV), dt_bias.to(DEV),
                          kd ** -0.5, 1e-6, q, k, v, gb, mode="channel_decay", decay_in=a_in.to(DEV), gk=gk)
        for i, (lo, n, skip) in enumerate([(0, 9, 0), (9, 5, 6)]):
            c = conv(seqs[i], None)[skip:]
            rq, rk = c[:, :qk].view(n, kvh, kd), c[:, qk:2 * qk].view(n, kvh, kd)
            rq = rq / torch.sqrt((rq * rq).sum(-1, keepdim=True) + 1e-6) * kd ** -0.5
            rk = rk / torch.sqrt((rk * rk).sum(-1, keepdim=True) + 1e-6)
            close(q[lo:lo + n].view(n, kvh, kd), rq, torch.float32, what="unit queries")
            close(k[lo:lo + n].view(n, kvh, kd), rk, torch.float32, what="unit keys")
            close(v[lo:lo + n], c[:, 2 * qk:], torch.float32, what="values")
            close(gb[lo:lo + n, :, 1], torch.sigmoid(seqs[i][skip:, ch:ch + heads].double()), torch.float32, what="step sizes")
            want = torch.exp(-torch.exp(a_log.double())[None, :, None] * pg.softplus(a_in[lo:lo + n].double() + dt_bias.double()).view(n, heads, kd))
            close(gk[lo:lo + n].view(n, heads, kd), want, torch.float32, what="decays per channel")
        # the state-space form: channels [v | k | q], a bias, no unit vectors, dt = softplus, decay from dt
        dt_b = torch.randn(heads, generator=g)
        ops.delta_prepare(proj.to(DEV), w_taps.to(DEV), kept, b, heads, kvh, kd, vd, ch, ch, a_log.to(DEV), dt_b.to(DEV),
                          1.0, 0.0, q, k, v, gb, mode="state_space", conv_bias=bias.to(DEV))
        for i, (lo, n, skip) in enumerate([(0, 9, 0), (9, 5, 6)]):
            c = conv(seqs[i], bias.double())[skip:]
            close(v[lo:lo + n], c[:, :vg], torch.float32, what="state-space values")
            close(k[lo:lo + n], c[:, vg:vg + qk], torch.float32, what="state-space keys")
            close(q[lo:lo + n], c[:, vg + qk:], torch.float32, what="state-space queries")
            dt = pg.softplus(seqs[i][skip:, ch:ch + heads].double() + dt_b.double())
            close(gb[lo:lo + n, :, 1], dt, torch.float32, what="step sizes")
            close(gb[lo:lo + n, :, 0], torch.exp(-torch.exp(a_log.double()) * dt), torch.float32, what="decays")
        ops.conv_state_update(proj.to(DEV), kept, b, taps, ch)
        if taps > 1:
            for i, slot in enumerate([1, 0]):
                tail = seqs[i][-(taps - 1):, :ch] if seqs[i].shape[0] >= taps - 1 else \
                    torch.cat([torch.zeros(taps - 1 - seqs[i].shape[0], ch), seqs[i][:, :ch]])
                assert torch.equal(kept[slot].cpu(), tail)
