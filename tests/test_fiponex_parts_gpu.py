"""Each new mechanism alone on the GPU against the plain implementation: the embedding scale, the norm with a weight
around zero and its adding form, the ReLU gate, the softmax router, biases / head norms / query stretch with the cache
write, the latent's norm and pairwise rotation with the cache write, the sigmoid gates, attention with a sink (planted
keys far back, at page borders, just inside and just outside the window, on the first positions; a sink that takes
nearly all the weight), and the gated delta rule (filters from kept inputs, unit norms, decays, the recurrence from a
state for unequal requests, and the same bits however a sequence is cut)."""
from types import SimpleNamespace

import pytest
import torch

import plain_fiponex as pf

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def close(got, ref, dtype, f32=2e-5, what=""):
    tol = f32 * max(1.0, float(ref.abs().max())) if dtype == torch.float32 else 2.0 ** -7 * float(ref.abs().max())
    worst = float((got.double().cpu() - ref.double()).abs().max())
    assert worst <= tol, (what, worst, tol)


def test_embedding_scale():
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(1)
    for dtype in DTYPES:
        table = torch.randn(50, 72, generator=g).to(dtype)
        tokens = [3, 49, 0, 3, 17]
        out = torch.empty(5, 72, device=DEV)
        ops.embedding(i32(tokens), table.to(DEV), out, scale=7.25)
        assert torch.equal(out.cpu(), table[tokens].float() * 7.25)
        ops.embedding(i32(tokens), table.to(DEV), out)
        assert torch.equal(out.cpu(), table[tokens].float())


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_with_a_weight_around_zero_and_its_adding_form(dtype):
    from tiny_llm_b200.engine import Workspace
    from tiny_llm_b200.parts import RMSNorm
    g = torch.Generator().manual_seed(2)
    for n, h, eps in [(5, 64, 1e-5), (33, 200, 1e-6), (3, 50, 1e-3)]:
        x = torch.randn(n, h, generator=g) * 3
        w = torch.randn(h, generator=g) * 0.2
        norm = RMSNorm(h, eps, weight_suffix="", one_plus=True)
        norm.load("n", {"n": w.to(DEV)})
        ctx = SimpleNamespace(workspace=Workspace(torch.device(DEV)), dtype=dtype)
        ref = pf.norm_one_plus(x.double(), w.double(), eps)
        close(norm.forward(ctx, x.to(DEV)), ref, dtype, what="one-plus norm")
        resid = torch.randn(n, h, generator=g)
        branch, stream = x.to(DEV), resid.to(DEV)
        norm.add_into(ctx, branch, stream)
        close(stream, resid.double() + ref, torch.float32, what="normed branch added")
        assert float(branch.abs().max()) == 0.0     # the branch buffer is handed back zeroed


@pytest.mark.parametrize("dtype", DTYPES)
def test_relu_gate(dtype):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(3)
    for m, inter, block in [(7, 96, 32), (130, 40, 8), (2, 6, 6)]:
        gu = torch.randn(m, 2 * inter, generator=g).to(dtype)
        out = torch.empty(m, inter, dtype=dtype, device=DEV)
        ops.silu_mul(gu.to(DEV), out, block, act="relu")
        v = gu.float().view(m, inter // block, 2, block)
        ref = (torch.relu(v[:, :, 0]) * v[:, :, 1]).reshape(m, inter)
        close(out, ref, dtype, what="relu gate")
        ops.silu_mul(gu.to(DEV), out, block)
        close(out, (pf.silu(v[:, :, 0]) * v[:, :, 1]).reshape(m, inter), dtype, what="silu gate")


def test_softmax_router():
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(4)
    for t, n, top in [(9, 6, 2), (70, 40, 5), (3, 3, 3), (5, 7, 1)]:
        z = torch.randn(t, n + 2, generator=g) * 2     # further columns of the row are not the router's
        z[0, 1] = z[0, 0]                              # a tie: the lower index wins
        ids = torch.empty(t, top, dtype=torch.int32, device=DEV)
        w = torch.empty(t, top, device=DEV)
        ops.moe_route(z.to(DEV), n, None, 1.0, ids, w, softmax=True)
        ref_ids, ref_w = pf.route_softmax(z[:, :n], top)
        assert torch.equal(ids.cpu().long(), ref_ids)
        assert float((w.cpu() - ref_w).abs().max()) <= 1e-6
        assert top == n or float(w.sum(dim=1).max()) < 1.0     # the chosen scores are not renormalised


@pytest.mark.parametrize("dtype", DTYPES)
def test_biases_head_norms_query_stretch_and_cache_write(dtype):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(5)
    for nq, nkv, kd, vd, page, every, coef in [(4, 2, 16, 24, 4, 8, 0.4), (6, 3, 10, 6, 8, 1, 0.25), (3, 1, 40, 40, 4, 0, 0.0)]:
        positions = [0, 1, 6, 7, 8, 15, 16, 700, 31999]
        t = len(positions)
        slots = [8, 9, 10, 20, 21, 1, 2, 3, 15]
        extra = 5      # columns behind q, k, v (a gate's) that the kernel must leave alone
        width = (nq + nkv) * kd + nkv * vd
        proj = torch.randn(t, width + extra, generator=g).to(dtype)
        bq, bk, bv = (torch.randn(n, generator=g) for n in (nq * kd, nkv * kd, nkv * vd))
        wq, wk = torch.rand(kd, generator=g) + 0.5, torch.rand(kd, generator=g) + 0.5
        kc = torch.zeros(6, nkv, page, kd, dtype=dtype, device=DEV)
        vc = torch.zeros(6, nkv, page, vd, dtype=dtype, device=DEV)
        dev = proj.to(DEV)
        eps = 1e-5
        ops.qk_norm_kv_write(dev, i32(positions), nq, nkv, kd, vd, kc, vc, i32(slots), bq.to(DEV), bk.to(DEV), bv.to(DEV),
                             wq.to(DEV), wk.to(DEV), eps=eps, stretch_coef=coef, stretch_every=every)
        src = proj.double()
        q = pf.norm_plain(src[:, :nq * kd].view(t, nq, kd) + bq.double().view(nq, kd), wq.double(), eps)
        if every:
            q = q * pf.query_stretch(torch.tensor(positions), coef, every)[:, None, None]
        k = pf.norm_plain(src[:, nq * kd:(nq + nkv) * kd].view(t, nkv, kd) + bk.double().view(nkv, kd), wk.double(), eps)
        v = src[:, (nq + nkv) * kd:width].view(t, nkv, vd) + bv.double().view(nkv, vd)
        got = dev.cpu()
        close(got[:, :nq * kd].view(t, nq, kd), q, dtype, what="queries")
        assert torch.equal(got[:, nq * kd:], proj[:, nq * kd:])     # nothing but the queries is rewritten in the row
        for i, s in enumerate(slots):
            close(kc[s // page, :, s % page], k[i], dtype, what="keys")
            close(vc[s // page, :, s % page], v[i], dtype, what="values")
        written = torch.zeros(6 * page, dtype=torch.bool)
        written[slots] = True
        assert float(kc.float().abs().sum(dim=(1, 3)).flatten().cpu()[~written].max()) == 0.0
    # the stretch steps up exactly where floor((p + 1) / every) does
    st = pf.query_stretch(torch.tensor([6, 7, 14, 15]), 0.4, 8)
    assert float(st[0]) == 1.0 and float(st[1]) > 1.0 and float(st[2]) == float(st[1]) and float(st[3]) > float(st[2])


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_norm_pairwise_rotation_and_cache_write(dtype):
    from tiny_llm_b200 import ops
    from tiny_llm_b200.parts import pair_frequencies
    g = torch.Generator().manual_seed(6)
    for nq, nd, rd, rank, rot, base, page in [(3, 16, 16, 32, 16, 100.0, 4), (5, 6, 10, 18, 10, 30.0, 8), (2, 12, 4, 9, 2, 10.0, 4),
                                              (1, 8, 8, 40, 0, 1.0, 4)]:
        positions = [0, 1, 2, 700, 701, 5, 6, 7, 31999]
        t = len(positions)
        slots = [8, 9, 10, 20, 21, 1, 2, 3, 15]
        kd = rank + rd
        proj = torch.randn(t, nq * (nd + rd) + kd + nq, generator=g).to(dtype)
        w = torch.rand(rank, generator=g) + 0.5
        kc = torch.zeros(6, 1, page, kd, dtype=dtype, device=DEV)
        vc = torch.zeros(6, 1, page, rank, dtype=dtype, device=DEV)
        q_out = torch.zeros(t, nq, kd, dtype=dtype, device=DEV)
        freq = pair_frequencies(rot, base).to(DEV) if rot else None
        ops.latent_kv_write(proj.to(DEV), i32(positions), nq, nd, rd, rank, rot, freq, w.to(DEV), 1e-5, q_out, kc, vc, i32(slots))
        src, pos = proj.double(), torch.tensor(positions)
        q = src[:, :nq * (nd + rd)].view(t, nq, nd + rd)
        lat = src[:, nq * (nd + rd):nq * (nd + rd) + kd]
        c = pf.norm_plain(lat[:, :rank], w.double(), 1e-5)
        k_rot = pf.rotate_pairs(lat[:, rank:].view(t, 1, rd), pos, rot, base, angles32=True)[:, 0]
        q_rot = pf.rotate_pairs(q[..., nd:], pos, rot, base, angles32=True)
        f32 = 2e-5
        close(q_out[..., rank:], q_rot, dtype, f32, "rotated query parts")
        assert float(q_out[..., :rank].float().abs().max()) == 0.0      # the plain parts are another kernel's
        if rot < rd:
            assert torch.equal(q_out[..., rank + rot:].cpu().double(), q[..., nd + rot:])     # what is not rotated passes
        for i, s in enumerate(slots):
            close(kc[s // page, 0, s % page, :rank], c[i], dtype, what="latent in the key row")
            close(kc[s // page, 0, s % page, rank:], k_rot[i], dtype, f32, "rotated key part")
            assert torch.equal(vc[s // page, 0, s % page], kc[s // page, 0, s % page, :rank])


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_product_per_head_in_one_launch(dtype):
    """Heads side by side in wider rows, inputs and outputs at offsets of their own; sizes the tensor-core tiles take
    and sizes they do not (odd K, odd offsets), one token and several row tiles; a row's bits do not depend on the
    rows beside it."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(11)
    for t, heads, k, n, a_pad, o_pad, a_off in [(1, 3, 16, 24, 8, 4, 0), (130, 2, 64, 192, 32, 0, 8), (70, 5, 6, 18, 10, 3, 1),
                                                (9, 1, 9, 7, 0, 0, 0), (33, 4, 40, 100, 2, 6, 2)]:
        wide = torch.randn(t, a_off + heads * (k + a_pad) + 6, generator=g).to(dtype).to(DEV)
        a = wide[:, a_off:a_off + heads * (k + a_pad)].view(t, heads, k + a_pad)[:, :, :k]
        w = (torch.randn(heads, n, k, generator=g) * 0.3).to(dtype).to(DEV)
        ref = torch.einsum("thk,hnk->thn", a.double().cpu(), w.double().cpu())
        for out_dtype in {dtype, torch.float32}:
            full = torch.full((t, heads, n + o_pad), 7.0, dtype=out_dtype, device=DEV)
            ops.head_linear(a, w, full[:, :, :n])
            close(full[:, :, :n], ref, out_dtype if out_dtype == torch.bfloat16 else torch.float32,
                  f32=2e-5 if dtype == torch.float32 else 1e-5, what=f"{heads} products of {k} -> {n}")
            if o_pad:
                assert float((full[:, :, n:].float() - 7.0).abs().max()) == 0.0      # nothing written beside the outputs
            alone = torch.empty(1, heads, n, dtype=out_dtype, device=DEV)
            ops.head_linear(a[t - 1:], w, alone)
            assert torch.equal(alone[0], full[t - 1, :, :n])


@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_gates_per_value_and_per_head(dtype):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(7)
    for t, heads, vd in [(7, 3, 40), (130, 2, 96), (1, 5, 7)]:
        x = torch.randn(t, heads * vd, generator=g)
        for cols in (heads * vd, heads):
            wide = torch.randn(t, cols + 11, generator=g).to(dtype)     # the gate is a slice of a wider row
            out = torch.empty(t, heads * vd, dtype=dtype, device=DEV)
            ops.sigmoid_gate(x.to(DEV), wide.to(DEV)[:, 3:3 + cols], heads, vd, out)
            gate = torch.sigmoid(wide[:, 3:3 + cols].double())
            gate = gate if cols == heads * vd else gate.repeat_interleave(vd, dim=1)
            close(out, x.double() * gate, dtype, what=f"gate of {cols} columns")


def paged(rows, table, page, pages):
    """rows [T, heads, d] -> cache [pages, heads, page, d] with position j in page table[j // page]."""
    t, heads, d = rows.shape
    cache = torch.full((pages, heads, page, d), float("nan"), dtype=rows.dtype)
    for j in range(t):
        cache[table[j // page], :, j % page] = rows[j]
    return cache


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page,length", [(None, 16, 700), (150, 16, 620), (24, 8, 100), (3, 4, 50), (20, 16, 300)])
def test_sink_attention_sees_exactly_the_window_and_finds_a_planted_key(dtype, window, page, length):
    """Keys are small but for one planted key per query position whose score stands out; it lies far back, at a page
    border, on the first position the window keeps (visible) or right before it (not visible).  Whether the kernel
    followed it shows in the output, which is then that key's value row (less the sink's share) or not.  Head 1's sink
    is so large that the head's output nearly vanishes; head 2's so small that it changes nothing."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(5)
    heads, kvh, kd, vd = 4, 2, 16, 32
    group = heads // kvh
    k = torch.randn(length, kvh, kd, generator=g) * 0.05
    v = torch.randn(length, kvh, vd, generator=g)
    pages_needed = -(-length // page)
    table = torch.randperm(pages_needed + 3, generator=g)[:pages_needed].tolist()
    qpos = sorted({length - 1, 0, 1, 2, page - 1, page, length // 2, length - 2} |
                  ({window - 1, window, window + 1} if window else set()))
    qpos = [p for p in qpos if 0 <= p < length][:kd]
    plants = {}
    q = torch.randn(len(qpos), heads, kd, generator=g) * 0.05
    for i, p in enumerate(qpos):
        first = max(0, p - window + 1) if window else 0
        inside = [first, (p // page) * page if (p // page) * page >= first else p, max(first, p - 3)]
        outside = [first - 1] if first > 0 else []
        target = (inside + outside)[(i + 1) % (len(inside) + len(outside))]
        plants[p] = target
        direction = torch.zeros(kd)
        direction[i] = 1.0     # one axis per query position: a key planted for one query says nothing to another
        k[target, 0] += 6.0 * direction
        for h in range(group):
            q[i, h] += 6.0 * direction
    sink = torch.tensor([0.5, 200.0, -60.0, 1.5])
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scale = 1.7
    kc, vc = paged(k, table, page, pages_needed + 3).to(DEV), paged(v, table, page, pages_needed + 3).to(DEV)
    bt = i32([table + [-1] * 5])
    kp = torch.arange(length)
    ref = torch.stack([pf.sink_softmax_attention(q[i:i + 1].double(), k.double(), v.double(), torch.tensor([p]), kp, scale,
                                                 sink.double(), window)[0] for i, p in enumerate(qpos)])
    no_sink = torch.stack([pf.sink_softmax_attention(q[i:i + 1].double(), k.double(), v.double(), torch.tensor([p]), kp, scale,
                                                     torch.full((heads,), -1e4, dtype=torch.float64), window)[0]
                           for i, p in enumerate(qpos)])
    for i, p in enumerate(qpos):       # the planted key decides head 0 (before the sink's share) exactly when it is visible
        visible = plants[p] <= p and (not window or p - plants[p] < window)
        near = float((no_sink[i, 0] - v[plants[p], 0].double()).abs().max()) < 0.05
        assert near == visible, (p, plants[p])
    assert float(ref[:, 1].abs().max()) < 1e-8 and float((ref[:, 2] - no_sink[:, 2]).abs().max()) < 1e-12
    assert float((ref[:, 3] - no_sink[:, 3]).abs().max()) > 1e-2       # a sink of ordinary size takes its share
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7 * float(ref.abs().max())

    def run(rows, out_dtype, generic=False):
        """Every query position a request of its own with one token (as decoded tokens run), all on the same pages."""
        n = len(rows)
        positions = [qpos[i] for i in rows]
        batch = SimpleNamespace(token_request=i32(list(range(n))), positions=i32(positions), cu_q=i32(list(range(n + 1))),
                                q_start=i32(positions), num_requests=n, max_q_len=1)
        qrows = q[rows].reshape(n, -1)
        pad = torch.zeros(n, 40, dtype=dtype)     # the queries lie at the front of wider rows
        out = torch.empty(n, heads * vd, dtype=out_dtype, device=DEV)
        ops.force_generic = generic
        try:
            ops.paged_attention_maps(torch.cat([qrows, pad], dim=1).to(DEV), heads, kvh, 1, kd, vd, kc, vc,
                                     bt.repeat(n, 1).contiguous(), batch, out, scale, window, None, sink=sink.to(DEV))
        finally:
            ops.force_generic = False
        return out.float().cpu().view(n, heads, vd)

    everyone = list(range(len(qpos)))
    for generic in (True, False):      # the CUDA-core kernel, then (bfloat16 only) the tensor-core kernel
        together = run(everyone, torch.float32, generic)
        assert torch.isfinite(together).all()
        assert float((together - ref).abs().max()) <= tol, generic
        for i, p in enumerate(qpos):       # every position alone: another launch shape
            alone = run([i], torch.float32, generic)
            assert float((alone[0] - ref[i]).abs().max()) <= tol, (p, generic)
            if dtype == torch.float32:
                assert torch.equal(alone[0], together[i]), p
    if dtype == torch.bfloat16:
        same_type = run(everyone, torch.bfloat16)
        assert float((same_type - ref).abs().max()) <= 2.0 ** -7 * float(ref.abs().max())


@pytest.mark.parametrize("kd,vd,heads,kvh,window", [(16, 32, 4, 2, None), (128, 96, 6, 1, 150), (80, 48, 8, 1, None), (32, 16, 5, 5, 200)])
def test_decoded_tokens_with_the_keys_in_runs_match_one_run(kd, vd, heads, kvh, window):
    """A step of decoded tokens may walk a row tile's keys in several runs that a second kernel joins: the same
    softmax (sink included) up to 32-bit rounding, for contexts of one token, of less than a tile, and of many tiles,
    with runs that end up empty for the short ones."""
    from tiny_llm_b200 import ops
    from tiny_llm_b200.engine import Workspace
    g = torch.Generator().manual_seed(17)
    page, contexts = 16, [1, 40, 300, 700, 65]
    r = len(contexts)
    pages_per = -(-max(contexts) // page)
    table = torch.arange(r * pages_per, dtype=torch.int32).view(r, pages_per)
    kc = (torch.randn(r * pages_per, kvh, page, kd, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    vc = torch.randn(r * pages_per, kvh, page, vd, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(r, heads * kd + 8, generator=g).to(torch.bfloat16).to(DEV)
    sink = torch.randn(heads, generator=g).to(DEV)
    batch = SimpleNamespace(cu_q=i32(list(range(r + 1))), q_start=i32([c - 1 for c in contexts]), num_requests=r, max_q_len=1,
                            max_kv_len=1024, token_request=i32(list(range(r))), positions=i32([c - 1 for c in contexts]))
    one, runs = torch.empty(r, heads * vd, device=DEV), torch.empty(r, heads * vd, device=DEV)
    for sk in (sink, None):
        ops.paged_attention_maps(q, heads, kvh, 1, kd, vd, kc, vc, table.to(DEV), batch, one, 0.2, window, None, sink=sk)
        ws = Workspace(torch.device(DEV))
        before = ops.launches
        ops.paged_attention_maps(q, heads, kvh, 1, kd, vd, kc, vc, table.to(DEV), batch, runs, 0.2, window, None, sink=sk, workspace=ws)
        assert ops.launches - before == 1 and ws.buffers(), "the keys were not cut into runs"
        assert float((one - runs).abs().max()) <= 4e-6 * max(1.0, float(one.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kd,vd,heads,kvh,window,page", [(16, 32, 4, 2, 24, 8), (48, 32, 6, 1, 150, 16), (128, 96, 6, 1, None, 16),
                                                         (28, 18, 5, 1, 7, 4), (24, 40, 3, 3, 50, 16)])
def test_sink_attention_portions_of_unequal_requests(dtype, kd, vd, heads, kvh, window, page):
    """Three requests in one step: a portion that starts far inside a sequence and crosses window and page edges, a
    single decoded token, and a prompt from position 0; both kernels against the plain implementation."""
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(kd + vd)
    spans = [(130, 97), (211, 1), (0, 75)]                 # (first position, tokens) of each request in this step
    lengths = [a + n for a, n in spans]
    scale = 0.9 / kd ** 0.5 * 4
    tables = []
    total_pages = sum(-(-n // page) for n in lengths) + 2
    kc = torch.full((total_pages, kvh, page, kd), float("nan"), dtype=dtype)
    vc = torch.full((total_pages, kvh, page, vd), float("nan"), dtype=dtype)
    order = torch.randperm(total_pages, generator=g).tolist()
    ks, vs = [], []
    for n in lengths:
        k = (torch.randn(n, kvh, kd, generator=g) * 0.7).to(dtype)
        v = torch.randn(n, kvh, vd, generator=g).to(dtype)
        table = [order.pop() for _ in range(-(-n // page))]
        for j in range(n):
            kc[table[j // page], :, j % page] = k[j]
            vc[table[j // page], :, j % page] = v[j]
        ks.append(k), vs.append(v), tables.append(table)
    width = max(len(t) for t in tables) + 2
    bt = i32([t + [-1] * (width - len(t)) for t in tables])
    t_all = sum(n for _, n in spans)
    q = (torch.randn(t_all, heads, kd, generator=g) * 0.7).to(dtype)
    sink = torch.randn(heads, generator=g) * 2
    ref = torch.empty(t_all, heads, vd, dtype=torch.float64)
    row, cu, req_of, pos_of = 0, [0], [], []
    for r, (a, n) in enumerate(spans):
        ref[row:row + n] = pf.sink_softmax_attention(q[row:row + n].double(), ks[r].double(), vs[r].double(),
                                                     torch.arange(a, a + n), torch.arange(lengths[r]), scale, sink.double(), window)
        row += n
        cu.append(row)
        req_of += [r] * n
        pos_of += list(range(a, a + n))
    batch = SimpleNamespace(token_request=i32(req_of), positions=i32(pos_of), cu_q=i32(cu), q_start=i32([a for a, _ in spans]),
                            num_requests=len(spans), max_q_len=max(n for _, n in spans))
    tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7 * float(ref.abs().max())
    for generic in (True, False):
        out = torch.empty(t_all, heads * vd, dtype=torch.float32, device=DEV)
        ops.force_generic = generic
        try:
            ops.paged_attention_maps(q.reshape(t_all, -1).to(DEV), heads, kvh, 1, kd, vd, kc.to(DEV), vc.to(DEV), bt, batch,
                                     out, scale, window, None, sink=sink.to(DEV))
        finally:
            ops.force_generic = False
        got = out.cpu().view(t_all, heads, vd)
        assert torch.isfinite(got).all(), generic
        bad = ((got - ref).abs().amax(dim=(1, 2)) > tol).nonzero().flatten().tolist()
        assert not bad, (generic, [(req_of[i], pos_of[i]) for i in bad[:8]])


def delta_inputs(g, t, heads, kvh, kd, vd, taps, dtype):
    c = 2 * kvh * kd + heads * vd
    proj = (torch.randn(t, c + heads * vd + 2 * heads + 3, generator=g) * 1.5).to(dtype)
    w_taps = torch.randn(c, taps, generator=g) * 0.5
    a_log, dt_bias = torch.rand(heads, generator=g) * 3 - 2.5, torch.randn(heads, generator=g)
    return c, proj, w_taps, a_log, dt_bias


def delta_plain(proj, w_taps, a_log, dt_bias, heads, kvh, kd, vd, before, s0):
    """One request's tokens through the plain functions, from kept inputs `before` [taps - 1, C] and state s0."""
    c = 2 * kvh * kd + heads * vd
    t = proj.shape[0]
    x, kept = pf.short_conv(proj[:, :c].double(), w_taps.double(), before.double())
    x = pf.silu(x)
    q, k, v = x[:, :kvh * kd].view(t, kvh, kd), x[:, kvh * kd:2 * kvh * kd].view(t, kvh, kd), x[:, 2 * kvh * kd:].view(t, heads, vd)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * kd ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(heads // kvh, dim=1), k.repeat_interleave(heads // kvh, dim=1)
    off = c + heads * vd
    beta = torch.sigmoid(proj[:, off:off + heads].double())
    gdec = torch.exp(-torch.exp(a_log.double()) * pf.softplus(proj[:, off + heads:off + 2 * heads].double() + dt_bias.double()))
    o, s = pf.delta_rule(q, k, v, beta, gdec, s0.double())
    return o.reshape(t, heads * vd), s, kept


def run_delta(ops, proj, w_taps, a_log, dt_bias, heads, kvh, kd, vd, taps, state, kept, batch):
    t = proj.shape[0]
    c = 2 * kvh * kd + heads * vd
    q = torch.empty(t, kvh * kd, device=DEV)
    k = torch.empty(t, kvh * kd, device=DEV)
    v = torch.empty(t, heads * vd, device=DEV)
    gb = torch.empty(t, heads, 2, device=DEV)
    off = c + heads * vd
    ops.delta_prepare(proj, w_taps, kept, batch, heads, kvh, kd, vd, off, off + heads, a_log, dt_bias, kd ** -0.5, 1e-6, q, k, v, gb)
    ops.conv_state_update(proj, kept, batch, taps, c)
    out = torch.empty(t, heads * vd, device=DEV)
    ops.delta_rule_scan(q, k, v, gb, state, batch, heads, kvh, kd, vd, out)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,kd,vd,taps", [(4, 2, 16, 8, 4), (3, 3, 24, 40, 2), (2, 1, 6, 10, 1), (5, 1, 70, 20, 3),
                                                  (2, 2, 130, 33, 4), (2, 1, 48, 64, 4), (1, 1, 256, 9, 2), (3, 3, 32, 17, 3)])
def test_delta_rule_from_a_state_for_unequal_requests(dtype, heads, kvh, kd, vd, taps):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(heads * kd + vd)
    lens, slots = [1, 23, 2, 40, 9], [4, 0, 5, 2, 1]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    t = cu[-1]
    c, proj, w_taps, a_log, dt_bias = delta_inputs(g, t, heads, kvh, kd, vd, taps, dtype)
    state = torch.randn(6, heads, vd, kd, generator=g) * 0.3          # the engine keeps S transposed
    kept = (torch.randn(6, max(taps - 1, 1), c, generator=g)).to(dtype).float()
    state_dev, kept_dev = state.to(DEV), kept.to(DEV)
    batch = SimpleNamespace(cu_q=i32(cu), slots=i32(slots), num_requests=len(lens), max_q_len=max(lens),
                            token_request=i32([r for r, n in enumerate(lens) for _ in range(n)]))
    out = run_delta(ops, proj.to(DEV), w_taps.to(DEV), a_log.to(DEV), dt_bias.to(DEV), heads, kvh, kd, vd, taps, state_dev,
                    kept_dev, batch)
    for r, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        before = kept[slots[r]][:taps - 1] if taps > 1 else torch.zeros(0, c)
        o, s, kept_after = delta_plain(proj[a:b].float(), w_taps, a_log, dt_bias, heads, kvh, kd, vd, before,
                                       state[slots[r]].transpose(1, 2))
        tol = 2e-5 * max(1.0, float(o.abs().max()))
        assert float((out[a:b].double().cpu() - o).abs().max()) <= tol, r
        assert float((state_dev[slots[r]].cpu().double() - s.transpose(1, 2)).abs().max()) <= tol, r
        if taps > 1:
            assert torch.equal(kept_dev[slots[r]].cpu().double(), kept_after), r
    assert torch.equal(state_dev[3].cpu(), state[3]) and torch.equal(kept_dev[3].cpu(), kept[3])   # no request's slot


@pytest.mark.parametrize("heads,kvh,kd,vd,taps,t", [(3, 1, 20, 12, 4, 57), (2, 2, 100, 24, 3, 41), (2, 1, 64, 8, 2, 33)])
def test_delta_rule_in_portions_gives_the_same_bits(heads, kvh, kd, vd, taps, t):
    from tiny_llm_b200 import ops
    g = torch.Generator().manual_seed(3)
    c, proj, w_taps, a_log, dt_bias = delta_inputs(g, t, heads, kvh, kd, vd, taps, torch.float32)
    proj, w_taps, a_log, dt_bias = proj.to(DEV), w_taps.to(DEV), a_log.to(DEV), dt_bias.to(DEV)

    def run(cuts):
        state = torch.zeros(2, heads, vd, kd, device=DEV)
        kept = torch.zeros(2, taps - 1, c, device=DEV)
        outs = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            batch = SimpleNamespace(cu_q=i32([0, b - a]), slots=i32([1]), num_requests=1, max_q_len=b - a,
                                    token_request=i32([0] * (b - a)))
            outs.append(run_delta(ops, proj[a:b], w_taps, a_log, dt_bias, heads, kvh, kd, vd, taps, state, kept, batch))
        return torch.cat(outs), state, kept

    whole, s, kp = run([0, t])
    for cuts in ([0, 2, 3, 30, t], [0, 1, 2, 4, 5, 8, 9, 17, t], list(range(t + 1))):
        o2, s2, k2 = run(cuts)
        assert torch.equal(o2, whole) and torch.equal(s2, s) and torch.equal(k2, kp)
