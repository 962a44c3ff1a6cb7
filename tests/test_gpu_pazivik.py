"""The Pazivik parts on the GPU: each kernel against the plain float64 function of its mechanism,
then the model through the step function and through generation, against the plain model."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_pazivik as pp
import traces
from conftest import PAZIVIK_TINY

pytestmark = pytest.mark.gpu

F = torch.float64


@pytest.fixture(scope="module")
def ops():
    from llmserve_b200.ops import get_ops

    return get_ops("cuda")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32).cuda()


def batch(q_lens, starts, slots, tokens=None):
    """The step arrays of a ragged batch (sequence i: q_lens[i] rows from position starts[i])."""
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    host = SimpleNamespace(q_lens=np.asarray(q_lens, dtype=np.int32),
                           ctx_lens=(np.asarray(starts) + np.asarray(q_lens)).astype(np.int32))
    return SimpleNamespace(
        cu_q=i32(cu), ctx_lens=i32(host.ctx_lens), state_slots=i32(slots),
        token_seq=i32(np.repeat(np.arange(len(q_lens)), q_lens)),
        positions=i32(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, q_lens)])),
        token_ids=None if tokens is None else i32(tokens), host=host, decode_splits=0,
        max_decode_ctx=int(max([s + n for s, n in zip(starts, q_lens) if n == 1], default=0)))


def close(got, ref, tol, what=""):
    err = (got.double().cpu() - ref.double()).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    assert err <= bound, f"{what}: {err:.3e} > {bound:.3e}"


# ----------------------------------------------------------------------------- embedding terms
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,buckets,mp,mc", [(70, 97, 31, 5), (256, 1, 2, 3), (33, 5003, 999983, 1000003)])
def test_hashed_pair_rows_and_the_token_kept_between_steps(ops, dtype, W, buckets, mp, mc):
    """A request in three steps beside others: the first token takes the last row, the first row
    of a later step pairs with the token the step before left in the slot, a slot that another
    request used starts afresh; products of token and multiplier pass 2^31."""
    table = rnd(buckets + 1, W, seed=1).to(dtype)
    state = torch.full((5, 1), 123456, dtype=torch.int32).cuda()
    seqs = {0: [40000, 7, 7, 49999, 3, 12], 3: [9, 49999, 49998, 1]}  # slot -> tokens
    steps = [([3, 2], [0, 0], [0, 3]), ([1, 1], [3, 2], [0, 3]), ([2, 1], [4, 3], [0, 3])]
    for q_lens, starts, slots in steps:
        toks = sum((seqs[s][a : a + n] for n, a, s in zip(q_lens, starts, slots)), [])
        x = torch.zeros(sum(q_lens), W).cuda()
        ops.hashed_pair_add(x, table.cuda(), state, batch(q_lens, starts, slots, toks), buckets=buckets,
                            mul_previous=mp, mul_token=mc)
        at = 0
        for n, a, s in zip(q_lens, starts, slots):
            rows = pp.bigram_rows(seqs[s][: a + n], buckets, mp, mc)[a:]
            assert torch.equal(x[at : at + n].cpu(), table.float()[rows]), (a, s)
            assert int(state[s, 0]) == seqs[s][a + n - 1]
            at += n
    assert int(state[1, 0]) == 123456
    # another request on slot 3, from position 0: what the slot holds is not read
    x = torch.zeros(2, W).cuda()
    ops.hashed_pair_add(x, table.cuda(), state, batch([2], [0], [3], [5, 6]), buckets=buckets, mul_previous=mp,
                        mul_token=mc)
    assert torch.equal(x.cpu(), table.float()[pp.bigram_rows([5, 6], buckets, mp, mc)])


@pytest.mark.parametrize("W", [6, 33, 324])
def test_sinusoid(ops, W):
    i = torch.arange((W + 1) // 2, dtype=F)
    freq = (10000.0 ** (-2.0 * i / W)).float().cuda()
    pos = [0, 1, 2, 77, 1000, 4095]
    x = rnd(len(pos), W, seed=3)
    got = x.clone().cuda()
    ops.sinusoid_add(got, i32(pos), freq)
    ref = x.to(F) + pp.sinusoid(4096, W)[pos]
    close(got, ref, 3e-4, "rows")  # the angle is a float32 product: at position 4095 its last bit is 2e-4
    close(got[:4], ref[:4], 4e-6, "early rows")


# ----------------------------------------------------------------------------- the latent row
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,page_tokens", [(16, 8), (40, 16), (128, 32), (200, 4)])
def test_latent_write_norms_and_finds_the_page(ops, dtype, R, page_tokens):
    Rp = -(-R // 16) * 16
    q_lens, starts = [5, 1, 3], [page_tokens - 2, 2 * page_tokens - 1, 0]  # across a page's border, at its last place
    T, col0 = sum(q_lens), 24
    proj = rnd(T, col0 + R + 3, seed=R, scale=3.0)
    weight = 1 + rnd(R, seed=9, scale=0.3)
    pages = torch.full((12, 1, page_tokens, Rp), 7.0, dtype=dtype).cuda()
    tables = i32([[3, 9, 0], [5, 6, 0], [11, 0, 0]])
    st = batch(q_lens, starts, [0, 1, 2])
    ops.latent_write(proj.cuda(), col0, R, weight.cuda(), 1e-5, pages, st.positions, st.token_seq, tables)
    ref = pp.rms_norm(proj[:, col0 : col0 + R].to(F), weight.to(F), 1e-5)
    at = 0
    for s, (n, a) in enumerate(zip(q_lens, starts)):
        for t in range(n):
            p = a + t
            row = pages[int(tables[s, p // page_tokens]), 0, p % page_tokens].float().cpu()
            close(row[:R], ref[at + t], 1e-6 if dtype == torch.float32 else 4e-3, "row")
            assert bool((row[R:] == 0).all())  # the padding of a rank that is no multiple of 16
        at += n
    assert int((pages != 7.0).any(-1).sum()) == T  # nothing else was written


@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32, torch.float32),
                                    (torch.float32, torch.bfloat16, torch.bfloat16),
                                    (torch.bfloat16, torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("T,H,N,K", [(1, 1, 16, 8), (5, 3, 48, 20), (70, 2, 33, 65), (130, 4, 128, 64), (200, 3, 136, 72)])
def test_head_linear(ops, dtypes, T, H, N, K):
    """Every kernel that serves the shape (CUDA cores; for bfloat16 rows of whole 16-byte vectors
    also the tensor-core tiles and the weight-streaming kernel) against the plain product."""
    ta, tw, to = dtypes
    col0 = 8
    a = rnd(T, col0 + H * K + (5 if K % 8 else 16), seed=T).to(ta)
    w = rnd(H, N, K, seed=K).to(tw)
    ref = torch.einsum("thk,hnk->thn", a[:, col0 : col0 + H * K].to(F).view(T, H, K), w.to(F)).reshape(T, H * N)
    for kind in (None, 0, 1, 2):
        got = ops.head_linear(a.cuda(), col0, w.cuda(), to, kind=kind)
        close(got, ref, 1e-5 if to == torch.float32 else 6e-3, f"kernel {kind}")


# ----------------------------------------------------------------------------- attention with sinks
def latent_attention_case(ops, dtype, H, R, page_tokens, ctx, n_rows, window, sinks, scale, seed, sharp_key=None,
                          splits=0):
    """One sequence of ``ctx`` latent rows in shuffled pages; the last ``n_rows`` are this step's
    queries (one row: the single-token kernel, cut into ``splits`` partitions if given). With
    ``sharp_key`` the last query of every head is made to single out that key, whose row carries a
    large planted value: the output shows it if and only if the key is read."""
    c = rnd(ctx, R, seed=seed)
    q = rnd(n_rows, H, R, seed=seed + 1)
    if sharp_key is not None:
        c[sharp_key] = 0
        c[sharp_key, 0] = 50.0
        q[-1, :, :] = 0
        q[-1, :, 0] = 40.0 / (50.0 * scale)  # score 40 against scores near 0
    pages_needed = -(-ctx // page_tokens)
    order = torch.randperm(pages_needed + 3, generator=torch.Generator().manual_seed(seed))[:pages_needed]
    pages = torch.full((pages_needed + 4, 1, page_tokens, R), float("nan"), dtype=dtype)
    for j in range(ctx):
        pages[order[j // page_tokens], 0, j % page_tokens] = c[j].to(dtype)
    st = batch([n_rows], [ctx - n_rows], [0])
    st.decode_splits = splits
    plan = {k: torch.tensor(v).cuda() for k, v in ops.attention_plan(st.host, dtype, R).items()}
    got = ops.paged_attention(
        q.reshape(n_rows, H * R).to(dtype).cuda(), num_heads=H, num_kv_heads=1, head_dim=R, scale=scale,
        window=window, k_pages=pages.cuda(), v_pages=pages.cuda(), block_tables=i32(order[None].tolist()),
        page_tokens=page_tokens, step=st, plan=plan, sinks=None if sinks is None else sinks.cuda())
    cq, qq = c.to(dtype).to(F), q.to(dtype).to(F)
    ref = torch.zeros(n_rows, H, R, dtype=F)
    for h in range(H):
        scores = torch.full((ctx, ctx), 0.0, dtype=F)
        scores[ctx - n_rows :] = qq[:, h] @ cq.T * scale
        sink = sinks[h].to(F) if sinks is not None else torch.tensor(-1e30, dtype=F)
        ref[:, h] = (pp.windowed_sink_softmax(scores, window, sink) @ cq)[ctx - n_rows :]
    return got.float().view(n_rows, H, R), ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,page_tokens,window", [(5, 128, 16, 75), (3, 48, 8, 5), (1, 16, 32, 0), (9, 64, 16, 40),
                                                    (2, 256, 16, 33)])
@pytest.mark.parametrize("n_rows,splits", [(70, 0), (2, 0), (1, 1), (1, 3)])
def test_sinks_join_the_denominator(ops, dtype, H, R, page_tokens, window, n_rows, splits):
    ops.check_attention_shape(R, dtype, H, 1)
    sinks = torch.linspace(-2.0, 3.0, H)
    got, ref = latent_attention_case(ops, dtype, H, R, page_tokens, ctx=300, n_rows=n_rows, window=window,
                                     sinks=sinks, scale=0.6 / R ** 0.5, seed=H + R, splits=splits)
    close(got, ref, 2e-5 if dtype == torch.float32 else 2e-2)
    # a large sink takes nearly all the weight: leaving it out would show at once
    big = torch.full((H,), 30.0)
    got, ref = latent_attention_case(ops, dtype, H, R, page_tokens, ctx=300, n_rows=n_rows, window=window,
                                     sinks=big, scale=0.6 / R ** 0.5, seed=H + R, splits=splits)
    assert float(ref.abs().max()) < 1e-6 and float(got.abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_rows,splits", [(40, 0), (1, 1), (1, 4)])
@pytest.mark.parametrize("edge", ["just outside", "just inside", "far inside", "first of the sequence"])
def test_a_key_at_the_windows_edge(ops, dtype, n_rows, splits, edge):
    """The last query's window of 100 reaches back to key ctx - 100, in the middle of a page; with
    no window, the very first key among hundreds is read."""
    ctx, window = 437, 100
    key = {"just outside": ctx - 101, "just inside": ctx - 100, "far inside": ctx - 50, "first of the sequence": 0}[edge]
    w = 0 if edge == "first of the sequence" else window
    got, ref = latent_attention_case(ops, dtype, 4, 128, 16, ctx=ctx, n_rows=n_rows, window=w,
                                     sinks=torch.tensor([0.5, -1.0, 2.0, 0.0]), scale=0.1, seed=7,
                                     sharp_key=key, splits=splits)
    close(got, ref, 3e-5 if dtype == torch.float32 else 2e-2)
    seen = ref[-1].abs().max() > 40  # the planted value is 50
    assert bool(seen) == (edge != "just outside")


# ----------------------------------------------------------------------------- routed experts
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,E,top,ff,shared", [(1, 70, 4, 4, 10, True), (37, 96, 5, 2, 24, False),
                                                 (150, 128, 16, 3, 48, True), (9, 64, 40, 1, 33, True),
                                                 (300, 32, 3, 1, 8, False), (700, 192, 6, 2, 136, True)])
def test_routed_experts_against_the_plain_sum(ops, dtype, T, W, E, top, ff, shared):
    h = rnd(T, W, seed=T).to(dtype)
    router = rnd(E + (1 if shared else 0), W, seed=1, scale=0.3)
    gu = rnd(E, 2 * ff, W, seed=2, scale=0.2).to(dtype)
    down = rnd(E, W, ff, seed=3, scale=0.2).to(dtype)
    shared_out = rnd(T, W, seed=4) if shared else None
    idx, wts, gate = ops.moe_route(h.cuda(), router.cuda(), E, top, shared)
    z = torch.sigmoid(h.to(F) @ router.to(F).T)
    val, ref_idx = torch.topk(z[:, :E], top, dim=-1)
    assert torch.equal(idx.cpu().long(), ref_idx)  # largest first (no two scores of a row are close)
    close(wts, val, 1e-6)
    if shared:
        close(gate, z[:, E], 1e-6)
    ref = torch.zeros(T, W, dtype=F)
    for t in range(T):
        for k in range(top):
            e = int(ref_idx[t, k])
            xin = val[t, k] * h[t].to(F)
            gg = gu[e].to(F) @ xin
            ref[t] += down[e].to(F) @ (pp.silu(gg[:ff]) * gg[ff:])
        if shared:
            ref[t] += z[t, E] * shared_out[t].to(F)
    n = T * top
    kinds = [None, 0] if dtype == torch.float32 else [None, 0, 1, 2] + ([3] if W % 8 == 0 and ff % 8 == 0 else [])
    for kind in kinds:  # every kernel of the experts' products gives the same sum
        plan = ops.moe_sort(idx, E, dtype, width=8 if W % 8 == 0 and ff % 8 == 0 else 1, kind=kind)
        work = plan.work
        offsets = work[: E + 1].cpu()
        perm, pos_of = work[E + 1 : E + 1 + n].cpu().long(), work[E + 1 + n : E + 1 + 2 * n].cpu().long()
        assert offsets[0] == 0 and offsets[-1] == n
        assert torch.equal(torch.bincount(idx.cpu().flatten().long(), minlength=E), offsets[1:] - offsets[:-1])
        assert torch.equal(pos_of[perm], torch.arange(n)) and sorted(perm.tolist()) == list(range(n))
        sorted_experts = idx.cpu().flatten()[perm]
        assert bool((sorted_experts[1:] >= sorted_experts[:-1]).all())
        g = ops.expert_linear(h.cuda(), gu.cuda(), plan, top=top, wts=wts)
        a = ops.silu_mul(g, out_dtype=dtype, activation="silu")
        y = ops.expert_linear(a, down.cuda(), plan)
        x = rnd(T, W, seed=5)
        into = x.clone().cuda()
        assert ops.moe_combine(y, plan, top, None if not shared else shared_out.cuda(), gate, into) is None
        close(into, ref + x.to(F), 2e-5 if dtype == torch.float32 else 1.5e-2, f"kernel {kind}")
        alone = ops.moe_combine(y, plan, top, None if not shared else shared_out.cuda(), gate, None)
        close(alone, ref, 2e-5 if dtype == torch.float32 else 1.5e-2, f"kernel {kind}")
    ops.check_kernel_errors()


def test_router_ties_go_to_the_lower_index(ops):
    h = torch.zeros(3, 16)
    h[1, 0] = 1.0
    router = torch.zeros(6, 16)
    router[4, 0] = 2.0
    idx, wts, _ = ops.moe_route(h.cuda(), router.cuda(), 6, 3, False)
    assert idx.cpu().tolist() == [[0, 1, 2], [4, 0, 1], [0, 1, 2]]
    assert wts.cpu()[0].tolist() == [0.5, 0.5, 0.5]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_gelu(ops, dtype):
    gu = rnd(9, 2 * 52, seed=1, scale=2.0).to(dtype)
    got = ops.silu_mul(gu.cuda(), out_dtype=dtype, activation="gelu_tanh")
    ref = pp.gelu_tanh(gu[:, :52].to(F)) * gu[:, 52:].to(F)
    close(got, ref, 2e-6 if dtype == torch.float32 else 5e-3)


# ----------------------------------------------------------------------------- the model
def gpu_runner(folder, name, num_pages, dtype, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.ops import get_ops

    _, _, model = load_model(folder, dtype, "cuda", get_ops("cuda"), max_len)
    return ModelRunner(model, page_tokens=PAZIVIK_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs, max_num_batched_tokens=max_len)


LENGTHS = {"P1": [5, 70, 1, 33, 49, 126, 2], "P2": [2, 40, 9, 64, 17, 100], "P3": [3, 150, 18, 77, 230],
           "P4": [4, 60, 1, 45, 90]}
TOL = {"float32": (2e-4, 5e-5), "bfloat16": (0.0, 0.03)}  # (absolute, relative to the largest logit)


@pytest.fixture(scope="module")
def expected(pazivik_dirs):
    out = {}
    for name in PAZIVIK_TINY:
        reqs = traces.make_requests(LENGTHS[name], PAZIVIK_TINY[name]["config"]["vocab"], seed=5)
        out[name] = (reqs, {r: pp.model_logits(pazivik_dirs[name], t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P1", "P2", "P3", "P4"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(pazivik_dirs, expected, name, mode, dtype):
    reqs, exp = expected[name]
    pool_tokens = traces.tokens_needed(reqs)
    runner = gpu_runner(pazivik_dirs[name], name, pool_tokens // PAZIVIK_TINY[name]["page_tokens"], dtype)
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)
    assert runner.manager.usage() == 0.0
    runner.check_kernels()


def test_layers_one_by_one_in_float32(pazivik_dirs):
    """The residual stream after every layer against the plain model's (the add that a layer
    leaves pending for the next norm is carried out first)."""
    folder = pazivik_dirs["P1"]
    tokens = traces.make_requests([60], 211, seed=2)["r0"]
    cfg, w = pp.load(folder)
    _, after = pp.forward(tokens, w, cfg, return_layers=True)
    runner = gpu_runner(folder, "P1", 8, "float32")
    model, seen = runner.model, []
    for block in model.blocks:
        inner = block.forward

        def spy(x, pending, step, cache, inner=inner):
            x, pending = inner(x, pending, step, cache)
            if hasattr(pending, "resolve"):
                pending = pending.resolve()
            if pending is not None:
                x += pending
            seen.append(x.clone())
            return x, None

        block.forward = spy
    from llmserve_b200.engine.batch import StepEntry

    runner.run([StepEntry("a", tokens, [0])])
    assert len(seen) == len(cfg["layers"])
    for i, x in enumerate(seen):
        close(x, after[i], 2e-5, f"after layer {i}")


def test_float32_logits_do_not_depend_on_the_cut(pazivik_dirs, expected):
    """Every kernel of the float32 path computes a row from that row's sequence alone and in a
    fixed order (attention's context partitions and tiles aside), so the mixed schedule gives the
    whole prompts' logits to the last bits."""
    reqs, _ = expected["P1"]
    pool = traces.tokens_needed(reqs) // 16
    a = traces.replay(gpu_runner(pazivik_dirs["P1"], "P1", pool, "float32"), traces.whole(reqs))
    b = traces.replay(gpu_runner(pazivik_dirs["P1"], "P1", pool, "float32"), traces.mixed(reqs, seed=4))
    scale = max(v.abs().max().item() for v in a.values())
    assert max((a[k] - b[k]).abs().max().item() for k in a) <= 4e-6 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(pazivik_dirs, dtype):
    """300 tokens one by one from position 0: every window passes over decoded tokens and pages
    that a window has left are given back while the request lives."""
    reqs = traces.make_requests([300], 211, seed=21)
    exp = {r: pp.model_logits(pazivik_dirs["P1"], t) for r, t in reqs.items()}
    runner = gpu_runner(pazivik_dirs["P1"], "P1", 6, dtype)  # 96 tokens of room for 300
    got = traces.replay(runner, traces.decode_tail(reqs, tail=300))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)


def test_slots_and_pages_used_again(pazivik_dirs):
    """One state slot and just enough pages: every request runs on what the one before it left."""
    reqs = traces.make_requests([40, 37, 64, 3], 211, seed=8)
    exp = {r: pp.model_logits(pazivik_dirs["P1"], t) for r, t in reqs.items()}
    runner = gpu_runner(pazivik_dirs["P1"], "P1", 4, "float32", max_num_seqs=1)
    traces.compare(traces.replay(runner, traces.portions(reqs)), exp, atol=2e-4, rtol=2e-5)


# ----------------------------------------------------------------------------- generation
PROMPTS = [[5, 9, 100, 31, 7], list(range(40, 57)), [3] * 33, [100, 2], list(range(70))]


def llm(folder, name, dtype, **kw):
    from llmserve_b200 import LLM

    d = dict(dtype=dtype, block_size=PAZIVIK_TINY[name]["page_tokens"], num_kv_blocks=64, max_model_len=256,
             max_num_seqs=8)
    d.update(kw)
    return LLM(str(folder), **d)


def greedy(n):
    from llmserve_b200 import SamplingParams

    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


@pytest.mark.parametrize("name", ["P1", "P2"])
@pytest.mark.parametrize("kw", [dict(cuda_graphs=False), dict(cuda_graphs=True),
                                dict(cuda_graphs=True, max_num_batched_tokens=24),
                                dict(cuda_graphs=True, num_kv_blocks=14, max_num_batched_tokens=16)])
def test_greedy_float32_equals_plain_greedy(pazivik_dirs, name, kw):
    """Through the entry point: the scheduler's batches, captured steps (single tokens and padded
    steps with portions, whose padding rows live on the spare slot), preemption by recomputation."""
    m = llm(pazivik_dirs[name], name, "float32", **kw)
    outs = m.generate(PROMPTS, greedy(12))
    for o, p in zip(outs, PROMPTS):
        assert o.outputs[0].token_ids == pp.greedy(pazivik_dirs[name], p, 12), (kw, p)


def test_greedy_bfloat16_picks_tokens_the_plain_model_also_ranks_first(pazivik_dirs):
    outs = llm(pazivik_dirs["P1"], "P1", "bfloat16").generate(PROMPTS, greedy(10))
    for o, p in zip(outs, PROMPTS):
        gen = o.outputs[0].token_ids
        logits = pp.model_logits(pazivik_dirs["P1"], p + gen)[len(p) - 1 : -1]
        for t, row in zip(gen, logits):
            assert float(row.max() - row[t]) <= 0.03 * float(row.abs().max())
