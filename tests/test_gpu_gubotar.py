"""The Gubotar parts on the GPU: each kernel against the plain float64 function of its mechanism,
then the model through the step function and through generation, against the plain model."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_gubotar as pg
import traces
from conftest import GUBOTAR_TINY

pytestmark = pytest.mark.gpu

F = torch.float64


@pytest.fixture(scope="module")
def ops():
    from llmserve_b200.ops import get_ops

    return get_ops("cuda")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def batch(q_lens, starts, slots):
    """The step arrays of a ragged batch (sequence i: q_lens[i] rows from position starts[i])."""
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32).cuda()
    return SimpleNamespace(
        cu_q=i32(cu), ctx_lens=i32(np.asarray(starts) + np.asarray(q_lens)), state_slots=i32(slots),
        token_seq=i32(np.repeat(np.arange(len(q_lens)), q_lens)),
        positions=i32(np.concatenate([np.arange(s, s + n) for s, n in zip(starts, q_lens)])))


def close(got, ref, tol, what=""):
    err = (got.double().cpu() - ref.double()).abs().max().item()
    bound = tol * max(1.0, ref.abs().max().item())
    assert err <= bound, f"{what}: {err:.3e} > {bound:.3e}"


# ----------------------------------------------------------------------------- token shift
@pytest.mark.parametrize("W", [68, 256, 1030])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift(ops, W, dtype):
    """Portions, a single token, a first token on a slot that holds another request's row."""
    q_lens, starts, slots = [5, 1, 2, 1], [0, 7, 3, 0], [2, 0, 3, 1]
    x, mu = rnd(sum(q_lens), W, seed=1), torch.rand(W, generator=torch.Generator().manual_seed(2))
    state = rnd(5, W, seed=3)
    got_state = state.clone().cuda()
    got = ops.token_shift(x.cuda(), mu.cuda(), got_state, batch(q_lens, starts, slots), dtype)
    at = 0
    for n, start, slot in zip(q_lens, starts, slots):
        before = state[slot].to(F) if start else torch.zeros(W, dtype=F)
        # the plain function on [the row before; the rows]: its first output row is dropped
        ref = pg.token_shift(torch.cat([before[None], x[at : at + n].to(F)]), mu.to(F))[1:]
        close(got[at : at + n], ref, 1e-6 if dtype == torch.float32 else 4e-3, "rows")
        assert torch.equal(got_state[slot].cpu(), x[at + n - 1])
        at += n
    assert torch.equal(got_state[4].cpu(), state[4])


# ----------------------------------------------------------------------------- linear attention with decay
def linear_attention_reference(proj, H, dk, dv, decay, silu, rot, base, key_scale, start=0):
    T = proj.shape[0]
    p = proj.to(F)
    q, k = p[:, : H * dk].view(T, H, dk), p[:, H * dk : 2 * H * dk].view(T, H, dk)
    v = p[:, 2 * H * dk : 2 * H * dk + H * dv].view(T, H, dv)
    if silu:
        q, k, v = pg.silu(q), pg.silu(k), pg.silu(v)
    if rot:
        q = torch.stack([pg.rotate_partial(q[t], start + t, rot, base) for t in range(T)])
        k = torch.stack([pg.rotate_partial(k[t], start + t, rot, base) for t in range(T)])
    return pg.decayed_outer_product_scan(q, k * key_scale, v, torch.tensor(decay, dtype=F)).reshape(T, H * dv)


def rotary_tables(rot, base, n):
    ang = torch.outer(torch.arange(n, dtype=F), base ** (-2 * torch.arange(rot // 2, dtype=F) / rot))
    return ang.cos().float().cuda(), ang.sin().float().cuda()


@pytest.mark.parametrize("H,dk,dv,rot,silu", [(2, 16, 16, 0, False), (3, 20, 40, 8, True), (1, 48, 16, 48, False),
                                              (2, 64, 64, 32, True), (1, 128, 96, 0, False), (2, 256, 8, 0, True),
                                              (1, 33, 300, 0, False)])
def test_decay_linear_attention(ops, H, dk, dv, rot, silu):
    """A whole prompt (more than one chunk of the kernel) against the plain recurrence; the same
    prompt in short portions beside another request, through state slots; and token by token,
    which gives the bits of the short portions."""
    T, extra = 150, 11  # extra columns after q|k|v stand for the gate
    decay = [0.999, 0.9, 0.5][:H]
    proj = rnd(T, 2 * H * dk + H * dv + extra, seed=H + dk, scale=0.7)
    cos, sin = rotary_tables(rot, 1e4, 256) if rot else (None, None)
    kw = dict(num_heads=H, key_dim=dk, value_dim=dv, decay=torch.tensor(decay).cuda(),
              activation="silu" if silu else "none", key_scale=dk ** -0.5, cos=cos, sin=sin)
    ref = linear_attention_reference(proj, H, dk, dv, decay, silu, rot, 1e4, dk ** -0.5)
    state = torch.full((4, H, dv, dk), 1e4).cuda()  # stale contents that must never be read at position 0
    whole = ops.decay_linear_attention(proj.cuda(), state=state, step=batch([T], [0], [1]), **kw)
    close(whole, ref, 2e-5, "whole")
    # portions of the same request on slot 2, another request's rows on slot 0 in between
    other = rnd(140, proj.shape[1], seed=99)
    state2 = torch.full((4, H, dv, dk), -1e4).cuda()
    got, at, oat = [], 0, 0
    for n, m in [(33, 2), (2, 0), (1, 1), (1, 20), (64, 1), (49, 100)]:
        rows = [proj[at : at + n]] + ([other[oat : oat + m]] if m else [])
        step = batch([n] + ([m] if m else []), [at] + ([oat] if m else []), [2] + ([0] if m else []))
        out = ops.decay_linear_attention(torch.cat(rows).cuda(), state=state2, step=step, **kw)
        got.append(out[:n])
        at, oat = at + n, oat + m
    got = torch.cat(got)
    close(got, ref, 2e-5, "portions")
    close(state2[2], state[1].cpu(), 2e-5, "final state")
    assert bool((state2[3] == -1e4).all())
    state3 = torch.zeros(4, H, dv, dk).cuda()
    single = torch.cat([ops.decay_linear_attention(proj[t : t + 1].cuda(), state=state3, step=batch([1], [t], [3]), **kw)
                        for t in range(T)])
    assert torch.equal(single, got) and torch.equal(state3[3], state2[2])


def test_linear_attention_chunked_and_short_sequences_in_one_step(ops):
    """Three long portions (several chunks each, one continuing from a state) beside single tokens."""
    H, dk, dv = 2, 128, 128
    decay = [0.99, 0.9995]
    width = 2 * H * dk + H * dv
    kw = dict(num_heads=H, key_dim=dk, value_dim=dv, decay=torch.tensor(decay).cuda(), activation="none",
              key_scale=dk ** -0.5, cos=None, sin=None)
    seqs = [rnd(n, width, seed=10 + i, scale=0.5) for i, n in enumerate([300, 1, 129, 1, 450])]
    state = torch.full((6, H, dv, dk), 3e3).cuda()
    # the first 40 rows of sequence 4 and 7 rows of sequence 1 and 3 ran in an earlier step
    first = ops.decay_linear_attention(torch.cat([seqs[4][:40], rnd(7, width, seed=30), rnd(7, width, seed=31)]).cuda(),
                                       state=state, step=batch([40, 7, 7], [0, 0, 0], [4, 1, 3]), **kw)
    rows = torch.cat([seqs[0], seqs[1], seqs[2], seqs[3], seqs[4][40:]])
    out = ops.decay_linear_attention(rows.cuda(), state=state,
                                     step=batch([300, 1, 129, 1, 410], [0, 7, 0, 7, 40], [0, 1, 2, 3, 4]), **kw)
    close(out[:300], linear_attention_reference(seqs[0], H, dk, dv, decay, False, 0, 0, dk ** -0.5), 2e-5, "0")
    close(out[301:430], linear_attention_reference(seqs[2], H, dk, dv, decay, False, 0, 0, dk ** -0.5), 2e-5, "2")
    ref4 = linear_attention_reference(seqs[4], H, dk, dv, decay, False, 0, 0, dk ** -0.5)
    close(first[:40], ref4[:40], 2e-5, "4, first step")
    close(out[431:], ref4[40:], 2e-5, "4, continued")
    ref1 = linear_attention_reference(torch.cat([rnd(7, width, seed=30), seqs[1]]), H, dk, dv, decay, False, 0, 0, dk ** -0.5)
    close(out[300:301], ref1[7:], 2e-5, "1")


def test_linear_attention_keeps_a_key_from_far_away(ops):
    """One early key/value pair is made large; with a decay close to one it must still be most of
    the output 700 tokens later (and gone with a small decay)."""
    H, dk, dv, T = 2, 32, 32, 700
    proj = rnd(T, 2 * H * dk + H * dv, seed=5, scale=0.05)
    proj[3, H * dk : 2 * H * dk] = 4.0  # k_3
    proj[3, 2 * H * dk :] = 3.0  # v_3
    proj[T - 1, : H * dk] = 1.0  # the last query looks along k_3
    decay = [0.9995, 0.9]
    state = torch.zeros(2, H, dv, dk).cuda()
    kw = dict(num_heads=H, key_dim=dk, value_dim=dv, decay=torch.tensor(decay).cuda(), state=state,
              activation="none", key_scale=1.0, cos=None, sin=None)
    got = ops.decay_linear_attention(proj.cuda(), step=batch([T], [0], [0]), **kw)
    ref = linear_attention_reference(proj, H, dk, dv, decay, False, 0, 0, 1.0)
    close(got, ref, 2e-5)
    assert ref[-1, :dv].abs().min() > 100 and ref[-1, dv:].abs().max() < 5
    # the same through 650 single tokens after a prompt of 50
    state.zero_()
    outs = [ops.decay_linear_attention(proj[:50].cuda(), step=batch([50], [0], [1]), **kw)]
    for t in range(50, T):
        outs.append(ops.decay_linear_attention(proj[t : t + 1].cuda(), step=batch([1], [t], [1]), **kw))
    close(torch.cat(outs), ref, 2e-5, "token by token")


@pytest.mark.parametrize("N,group,weighted,gate", [(96, 32, False, "silu"), (80, 80, True, "sigmoid"),
                                                   (1200, 1200, True, "silu"), (48, 16, False, "sigmoid")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_group_norm(ops, N, group, weighted, gate, dtype):
    T, off, eps = 9, 37, 1e-5
    o, proj = rnd(T, N, seed=1, scale=3.0), rnd(T, off + N + 5, seed=2)
    w = rnd(N, seed=3) if weighted else None
    got = ops.gated_group_norm(o.cuda(), proj.cuda(), gate_offset=off, group=group,
                               weight=None if w is None else w.cuda(), eps=eps, gate_activation=gate, out_dtype=dtype)
    y = pg.rms(o.to(F).view(T, N // group, group), eps).reshape(T, N)
    if weighted:
        y = y * w.to(F)
    g = proj[:, off : off + N].to(F)
    ref = y * (pg.silu(g) if gate == "silu" else pg.sigmoid(g))
    close(got, ref, 2e-6 if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("H", [68, 256, 2500])
@pytest.mark.parametrize("two", [False, True])
@pytest.mark.parametrize("emit", [None, torch.float32, torch.bfloat16])
def test_rmsnorm_add_of_one_branch_and_of_two_normed_branches(ops, H, two, emit):
    from llmserve_b200.parts.base import BranchMix

    T, eps = 7, 1e-5
    x, a, b = rnd(T, H, seed=1), rnd(T, H, seed=2, scale=5.0), rnd(T, H, seed=3, scale=0.01)
    wa, wb, w = rnd(H, seed=4), rnd(H, seed=5), rnd(H, seed=6)
    if two:
        y = 0.5 * pg.rms(a.to(F), 1e-6) * wa.to(F) + 0.25 * pg.rms(b.to(F), 1e-6) * wb.to(F)
        branch = BranchMix(ops, [a.cuda(), b.cuda()], [wa.cuda(), wb.cuda()], (0.5, 0.25), 1e-6)
        close(branch.resolve(), y, 2e-6, "the sum alone")
    else:
        y, branch = a.to(F), a.cuda()
    ref = x.to(F) + pg.rms(y, eps) * w.to(F)
    gx = x.clone().cuda()
    out = ops.rmsnorm_add(gx, branch, w.cuda(), eps, out_dtype=emit)
    close(gx, ref, 2e-6, "x")
    if emit is None:
        assert out is None
    else:
        assert out.dtype == emit
        close(out, ref, 2e-6 if emit == torch.float32 else 4e-3, "emitted")


# ----------------------------------------------------------------------------- q/k norm and page write
@pytest.mark.parametrize("D,norm_dim,values_are_keys,rope", [(48, 40, True, False), (32, 32, False, True),
                                                              (16, 16, True, True), (128, 128, False, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_rotation_and_page_write(ops, D, norm_dim, values_are_keys, rope, dtype):
    from plain_ops import PlainOps

    nq, nk, page, eps = 4, 2, 8, 1e-5
    q_lens, starts = [5, 1, 3], [0, 20, 6]
    T = sum(q_lens)
    heads = nq + nk + (0 if values_are_keys else nk)
    qkv = rnd(T, heads * D, seed=1)
    if norm_dim < D:
        qkv.view(T, heads, D)[:, :, norm_dim:] = 0
    qw, kw_ = rnd(D, seed=2), rnd(D, seed=3)
    cos, sin = rotary_tables(D, 1e4, 64) if rope else (None, None)
    step = batch(q_lens, starts, [0, 1, 2])
    tables = torch.tensor([[3, 0, 9, 9], [4, 5, 6, 9], [1, 2, 9, 9]], dtype=torch.int32)
    kp = torch.full((10, nk, page, D), 7.0, dtype=dtype)
    vp = torch.full((10, nk, page, D), -7.0, dtype=dtype)
    kw = dict(num_heads=nq, num_kv_heads=nk, head_dim=D, norm_dim=norm_dim, values_are_keys=values_are_keys,
              eps=eps, page_tokens=page, out_dtype=dtype)
    kp_ref, vp_ref = kp.clone(), vp.clone()
    q_ref = PlainOps().norm_rope_kv_write(qkv, q_weight=qw, k_weight=kw_, positions=step.positions.cpu(),
                                          token_seq=step.token_seq.cpu(), cos=None if cos is None else cos.cpu(),
                                          sin=None if sin is None else sin.cpu(), k_pages=kp_ref, v_pages=vp_ref,
                                          block_tables=tables, **kw)
    kp_g, vp_g = kp.cuda(), vp.cuda()
    q_g = ops.norm_rope_kv_write(qkv.cuda(), q_weight=qw.cuda(), k_weight=kw_.cuda(), positions=step.positions,
                                 token_seq=step.token_seq, cos=cos, sin=sin, k_pages=kp_g, v_pages=vp_g,
                                 block_tables=tables.cuda(), **kw)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    close(q_g, q_ref.float(), tol, "q")
    close(kp_g, kp_ref.float(), tol, "k pages")
    close(vp_g, vp_ref.float(), tol, "v pages")
    # an independent look at one key: token 2 of the last sequence, key head 1
    t = 8
    k_raw = qkv[t].view(heads, D)[nq + 1, :norm_dim].to(F)
    want = pg.rms(k_raw, eps) * kw_[:norm_dim].to(F)
    if rope:
        want = pg.rotate_partial(want[None], 8, D, 1e4)[0]
    close(kp_g[2, 1, 0, :norm_dim], want, tol, "one key by hand")  # position 8: page 1 of the sequence, offset 0
    if values_are_keys:
        close(vp_g[2, 1, 0, :norm_dim], k_raw, tol, "the value is the key as projected")


# ----------------------------------------------------------------------------- attention with score options
def attention_case(ops, dtype, H, G, D, page, ctx, n_rows, chunk, temp, slopes, scale, seed, sharp_key=None):
    """The last ``n_rows`` positions of a context of ``ctx`` tokens are the queries; keys and
    values lie in shuffled pages. Returns (engine output, plain output)."""
    ops.check_attention_shape(D, dtype)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n_rows, H, D, generator=g).to(dtype)
    k = torch.randn(ctx, G, D, generator=g).to(dtype)
    v = torch.randn(ctx, G, D, generator=g).to(dtype)
    if sharp_key is not None:  # a key that every query would pick if it were visible
        q = (q.float() + 1.0).to(dtype)
        k[sharp_key] = 4.0
        v[sharp_key] = 50.0
    blocks = -(-ctx // page)
    order = torch.randperm(blocks + 2, generator=g)
    kp = torch.full((blocks + 2, G, page, D), 300.0).to(dtype)
    vp = torch.full((blocks + 2, G, page, D), -3e4).to(dtype)
    for j in range(ctx):
        kp[order[j // page], :, j % page] = k[j]
        vp[order[j // page], :, j % page] = v[j]
    host = SimpleNamespace(q_lens=np.array([n_rows]), ctx_lens=np.array([ctx]))
    plan = {kk: torch.from_numpy(vv).cuda() for kk, vv in ops.attention_plan(host, dtype, D).items()}
    step = SimpleNamespace(cu_q=torch.tensor([0, n_rows], dtype=torch.int32).cuda(),
                           ctx_lens=torch.tensor([ctx], dtype=torch.int32).cuda(), decode_splits=0,
                           max_decode_ctx=ctx if n_rows == 1 else 0)
    f32 = lambda a: None if a is None else torch.tensor(a, dtype=torch.float32).cuda()
    got = ops.paged_attention(q.view(n_rows, H * D).cuda(), num_heads=H, num_kv_heads=G, head_dim=D, scale=scale,
                              window=0, k_pages=kp.cuda(), v_pages=vp.cuda(),
                              block_tables=order[:blocks].to(torch.int32)[None].cuda(), page_tokens=page,
                              step=step, plan=plan, head_scale=f32(temp), slopes=f32(slopes), chunk=chunk)
    ref = pg.chunked_softmax(q.to(F), k.to(F), v.to(F), scale,
                             torch.tensor(temp if temp is not None else [1.0] * H, dtype=F),
                             torch.tensor(slopes if slopes is not None else [0.0] * H, dtype=F),
                             chunk if chunk else 1 << 30, start=ctx - n_rows)
    return got.view(n_rows, H, D), ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,page", [(4, 2, 16, 16), (3, 1, 48, 8), (6, 6, 64, 16), (8, 2, 128, 32)])
@pytest.mark.parametrize("n_rows", [1, 2, 150])
def test_attention_with_temperature_slopes_and_chunks(ops, dtype, H, G, D, page, n_rows):
    temp = [0.5 + 0.3 * h for h in range(H)]
    slopes = pg.head_slopes(H).tolist()
    got, ref = attention_case(ops, dtype, H, G, D, page, ctx=333, n_rows=n_rows, chunk=50, temp=temp,
                              slopes=slopes, scale=D ** -0.5, seed=D + n_rows)
    close(got, ref, 3e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("options", ["chunk", "slopes", "temperature"])
def test_each_score_option_alone(ops, dtype, options):
    H, D = 4, 32
    kw = dict(chunk=0, temp=None, slopes=None)
    if options == "chunk":
        kw["chunk"] = 37
    elif options == "slopes":
        kw["slopes"] = [0.5, 0.1, 0.02, 0.0]
    else:
        kw["temp"] = [2.0, 1.0, 0.25, -0.5]
    for n_rows in (1, 70):
        got, ref = attention_case(ops, dtype, H, 2, D, 16, ctx=200, n_rows=n_rows, scale=0.3, seed=3, **kw)
        close(got, ref, 3e-5 if dtype == torch.float32 else 2e-2, f"{options}, {n_rows} rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_rows", [1, 3, 140])
@pytest.mark.parametrize("edge", ["just outside", "just inside", "first of the sequence"])
def test_a_key_at_a_chunk_edge(ops, dtype, n_rows, edge):
    """A key that every query would pick is put just before the last chunk's first position (no
    query of that chunk may see it), on that position (all of them see it), or at position 0."""
    chunk, ctx = 48, 48 * 5 + 7  # the last chunk starts at 240, in the middle of a page of 32
    key = {"just outside": 239, "just inside": 240, "first of the sequence": 0}[edge]
    got, ref = attention_case(ops, dtype, 4, 2, 64, 32, ctx=ctx, n_rows=n_rows, chunk=chunk, temp=[1.0] * 4,
                              slopes=[0.0] * 4, scale=0.125, seed=7, sharp_key=key)
    close(got, ref, 3e-5 if dtype == torch.float32 else 2e-2)
    seen = ref[-1].abs().max() > 40  # the planted value is 50
    assert bool(seen) == (edge == "just inside")


# ----------------------------------------------------------------------------- the model
def gpu_runner(folder, name, num_pages, dtype, max_num_seqs=4, max_len=512):
    from llmserve_b200.engine.runner import ModelRunner, load_model
    from llmserve_b200.ops import get_ops

    _, _, model = load_model(folder, dtype, "cuda", get_ops("cuda"), max_len)
    return ModelRunner(model, page_tokens=GUBOTAR_TINY[name]["page_tokens"], num_pages=num_pages,
                       max_model_len=max_len, max_num_seqs=max_num_seqs, max_num_batched_tokens=max_len)


LENGTHS = {"G1": [5, 70, 1, 33, 49, 126, 2], "G2": [2, 40, 9, 64, 17, 100], "G3": [3, 50, 18, 77, 130], "G4": [5, 70, 33, 100, 1]}
TOL = {"float32": (0.0, 2e-5), "bfloat16": (0.0, 0.03)}  # (absolute, relative to the largest logit)


@pytest.fixture(scope="module")
def expected(gubotar_dirs):
    out = {}
    for name in GUBOTAR_TINY:
        reqs = traces.make_requests(LENGTHS[name], GUBOTAR_TINY[name]["config"]["vocab"], seed=5)
        out[name] = (reqs, {r: pg.model_logits(gubotar_dirs[name], t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["G1", "G2", "G3", "G4"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_every_way_of_cutting_matches_plain(gubotar_dirs, expected, name, mode, dtype):
    reqs, exp = expected[name]
    pool_tokens = traces.tokens_needed(reqs)
    runner = gpu_runner(gubotar_dirs[name], name, pool_tokens // GUBOTAR_TINY[name]["page_tokens"], dtype)
    got = traces.replay(runner, getattr(traces, mode)(reqs))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)
    assert runner.manager.usage() == 0.0
    runner.check_kernels()


def test_float32_logits_do_not_depend_on_the_cut(gubotar_dirs, expected):
    """Every kernel of the float32 path computes a row from that row's sequence alone and in a
    fixed order, so the mixed schedule gives the bits of the whole prompts (attention's context
    partitions and tiles aside)."""
    reqs, _ = expected["G1"]
    pool = traces.tokens_needed(reqs) // 16
    a = traces.replay(gpu_runner(gubotar_dirs["G1"], "G1", pool, "float32"), traces.whole(reqs))
    b = traces.replay(gpu_runner(gubotar_dirs["G1"], "G1", pool, "float32"), traces.mixed(reqs, seed=4))
    scale = max(v.abs().max().item() for v in a.values())
    assert max((a[k] - b[k]).abs().max().item() for k in a) <= 4e-6 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(gubotar_dirs, dtype):
    """300 tokens one by one from position 0, over several chunks of the attention."""
    reqs = traces.make_requests([300], 211, seed=21)
    exp = {r: pg.model_logits(gubotar_dirs["G1"], t) for r, t in reqs.items()}
    runner = gpu_runner(gubotar_dirs["G1"], "G1", 320 // 16, dtype)
    got = traces.replay(runner, traces.decode_tail(reqs, tail=300))
    atol, rtol = TOL[dtype]
    traces.compare(got, exp, atol=atol, rtol=rtol)


def test_slots_and_pages_used_again(gubotar_dirs):
    """One state slot and just enough pages: every request runs on what the one before it left."""
    reqs = traces.make_requests([40, 37, 64, 3], 211, seed=8)
    exp = {r: pg.model_logits(gubotar_dirs["G1"], t) for r, t in reqs.items()}
    runner = gpu_runner(gubotar_dirs["G1"], "G1", 4, "float32", max_num_seqs=1)
    traces.compare(traces.replay(runner, traces.portions(reqs)), exp, atol=0.0, rtol=2e-5)


# ----------------------------------------------------------------------------- generation
PROMPTS = [[5, 9, 100, 31, 7], list(range(40, 57)), [3] * 33, [100, 2], list(range(70))]


def llm(folder, name, dtype, **kw):
    from llmserve_b200 import LLM

    d = dict(dtype=dtype, block_size=GUBOTAR_TINY[name]["page_tokens"], num_kv_blocks=64, max_model_len=256,
             max_num_seqs=8)
    d.update(kw)
    return LLM(str(folder), **d)


def greedy(n):
    from llmserve_b200 import SamplingParams

    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


@pytest.mark.parametrize("name", ["G1", "G2"])
@pytest.mark.parametrize("kw", [dict(cuda_graphs=False), dict(cuda_graphs=True),
                                dict(cuda_graphs=True, max_num_batched_tokens=24),
                                dict(cuda_graphs=True, num_kv_blocks=14, max_num_batched_tokens=16)])
def test_greedy_float32_equals_plain_greedy(gubotar_dirs, name, kw):
    """Through the entry point: the scheduler's batches, captured steps (single tokens and padded
    steps with portions, whose padding rows live on the spare slot), preemption by recomputation."""
    m = llm(gubotar_dirs[name], name, "float32", **kw)
    outs = m.generate(PROMPTS, greedy(12))
    for o, p in zip(outs, PROMPTS):
        assert o.outputs[0].token_ids == pg.greedy(gubotar_dirs[name], p, 12), (kw, p)


def test_greedy_bfloat16_picks_tokens_the_plain_model_also_ranks_first(gubotar_dirs):
    outs = llm(gubotar_dirs["G1"], "G1", "bfloat16").generate(PROMPTS, greedy(10))
    for o, p in zip(outs, PROMPTS):
        gen = o.outputs[0].token_ids
        logits = pg.model_logits(gubotar_dirs["G1"], p + gen)[len(p) - 1 : -1]
        for t, row in zip(gen, logits):
            assert float(row.max() - row[t]) <= 0.03 * float(row.abs().max())
