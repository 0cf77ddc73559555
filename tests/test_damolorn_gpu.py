"""Damolorn on the GPU: every mechanism's kernel alone against the plain implementation
(``plain_damolorn``), the engine under every way of cutting the same requests, planted keys that
one score singles out (far back, at page borders, the newest key, the first key, and one past
the causal edge), convolution state and pages that change hands, long decoding, and greedy
generation through the entry point and its scheduler."""

from __future__ import annotations

import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_damolorn as plain
import replay_cases as rc
import tiny_damolorn as td

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
LENGTHS = {"dam_a": [1, 2, 9, 23, 40, 31, 130], "dam_b": [3, 17, 50, 8, 70, 33, 150],
           "dam_c": [2, 48, 11, 61, 35, 5, 97]}
TOL32 = 5e-5  # of the largest |logit|
TOL16 = 6e-2  # bfloat16, wide weights; a few positions may flip an expert (see _compare)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _K():
    from emberserve_b200 import kernels

    return kernels


@pytest.fixture(scope="module")
def dam_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("damolorn")
    return {name: td.write_model(cfg, root / name, td.SEEDS[name]) for name, cfg in td.ALL.items()}


# ---- mechanisms alone -------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("width,groups,post_groups", [(48, 3, 3), (64, 1, 4), (250, 2, 1), (4096, 8, 2)])
def test_grouped_norm_with_the_norm_of_what_joins_the_stream(dtype, width, groups, post_groups):
    K = _K()
    g = torch.Generator().manual_seed(width)
    n = 7
    res = torch.randn(n, width, generator=g) * 3
    delta = (torch.randn(n, width, generator=g) * 5).to(dtype)
    gain = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype)
    post = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    for case in ("none", "plain", "normed", "rows"):
        r_dev = res.to(DEV).clone()
        out = torch.empty(n if case != "rows" else 3, width, dtype=dtype, device=DEV)
        rows = _i32([5, 0, 2]) if case == "rows" else None
        d = None if case == "none" else delta.to(DEV)
        pg = post.to(DEV) if case in ("normed", "rows") else None
        K.add_norm_grouped(d, pg, post_groups, 1e-5, r_dev, gain.to(DEV), groups, 3e-6, out, rows=rows)
        want_res = res.double()
        if case == "plain":
            want_res = want_res + delta.double()
        elif case in ("normed", "rows"):
            want_res = want_res + plain.grouped_norm(delta.double(), post.double(), post_groups, 1e-5)
        want = plain.grouped_norm(want_res, gain.double(), groups, 3e-6)
        if case == "rows":
            want = want[[5, 0, 2]]
            assert torch.equal(r_dev.cpu(), res)  # the stream is left alone
        else:
            assert (r_dev.cpu().double() - want_res).abs().max() <= 1e-5 * want_res.abs().max()
        assert (out.cpu().double() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_causal_taps_in_steps_with_state_that_changes_hands(dtype, taps):
    """Two requests cut into portions of 1, 2 and more tokens (shorter than the taps reach), in one
    batch, through slots that held another request's inputs before."""
    K = _K()
    c = 24
    g = torch.Generator().manual_seed(taps)
    w = (torch.randn(c, taps, generator=g)).to(dtype)
    seqs = [torch.randn(13, c, generator=g).to(dtype), torch.randn(9, c, generator=g).to(dtype)]
    want = [plain.causal_taps(s.double(), w.double()) for s in seqs]
    state = torch.randn(4, max(taps - 1, 1), c, device=DEV) * 100 if taps > 1 else None  # stale contents
    slots = _i32([3, 1])
    if taps > 1:
        state[[3, 1]] = 0  # what the engine does with a slot that is handed out
    cuts = [[1, 2, 1, 4, 5], [2, 1, 1, 3, 2]]
    at = [0, 0]
    got = [[], []]
    for step in range(5):
        q = [cuts[0][step], cuts[1][step]]
        x = torch.cat([seqs[r][at[r]:at[r] + q[r]] for r in range(2)]).to(DEV)
        out = torch.empty_like(x)
        K.causal_taps(x, w.to(DEV), state, slots if taps > 1 else None, _i32([0, q[0], q[0] + q[1]]),
                      _i32([0] * q[0] + [1] * q[1]), out, 2)
        got[0].append(out[:q[0]].cpu())
        got[1].append(out[q[0]:].cpu())
        at = [at[0] + q[0], at[1] + q[1]]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for r in range(2):
        o = torch.cat(got[r]).double()
        assert (o - want[r]).abs().max() <= tol * want[r].abs().max()


@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("dims,rope_dim", [(8, 8), (4, 10), (2, 2)])
def test_rotation_pairings_in_the_query_and_in_the_cached_key(pairing, dims, rope_dim):
    K = _K()
    g = torch.Generator().manual_seed(dims)
    n, heads, nope, qr, r, base = 6, 3, 5, 7, 12, 300.0
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    table = K.rope_table(inv, 64)
    positions = [0, 1, 17, 33, 5, 63]
    # queries, in place
    q = torch.randn(n, heads * (nope + rope_dim), generator=g)
    q_dev = q.to(DEV).clone()
    K.rope_inplace(q_dev, heads, nope + rope_dim, nope, dims, pairing, _i32(positions), table)
    want = q.double().view(n, heads, nope + rope_dim).clone()
    want[..., nope:] = plain.rotate(want[..., nope:], base, dims, pairing, torch.tensor(positions))
    assert (q_dev.cpu().double().view(n, heads, -1) - want).abs().max() < 2e-5
    # the shared key part, on its way into the cache, beside the two latent norms
    proj = torch.randn(n, qr + r + rope_dim + 3, generator=g)
    qg, kg = 1 + 0.3 * torch.randn(qr, generator=g), 1 + 0.3 * torch.randn(r, generator=g)
    pages = torch.zeros(16, 4, r + rope_dim, device=DEV)
    bt = _i32([[3, 7, 1, 0, 9, 2, 4, 5, 6, 8, 10, 11, 12, 13, 14, 15]])
    cq = torch.empty(n, qr, device=DEV)
    K.latent_prep(proj.to(DEV), qr, r, rope_dim, qg.to(DEV), kg.to(DEV), 1e-5, _i32(positions), _i32([0] * n),
                  table, dims, pairing, pages, bt, cq)
    p64 = proj.double()
    assert (cq.cpu().double() - plain.rms(p64[:, :qr], 1e-5) * qg.double()).abs().max() < 1e-5
    c = plain.rms(p64[:, qr:qr + r], 1e-5) * kg.double()
    kr = plain.rotate(p64[:, qr + r:qr + r + rope_dim], base, dims, pairing, torch.tensor(positions))
    for i, pos in enumerate(positions):
        vec = pages[int(bt[0, pos // 4]), pos % 4].cpu().double()
        assert (vec - torch.cat((c[i], kr[i]))).abs().max() < 2e-5


def _latent_case(seed, dtype, heads, r, p, ctx_lens, q_lens, page_size):
    """Random cached vectors for requests with `ctx_lens` tokens in the cache, the last `q_lens`
    of which are the step's queries.  Returns the kernel's arguments and the dense answer."""
    g = torch.Generator().manual_seed(seed)
    rows = len(ctx_lens)
    width = max(-(-c // page_size) for c in ctx_lens)
    num_pages = rows * width + 3
    perm = torch.randperm(num_pages, generator=g)[:rows * width].view(rows, width)
    pages = (torch.randn(num_pages, page_size, r + p, generator=g) * 50).to(dtype)  # stale pages hold large numbers
    vecs = [torch.randn(c, r + p, generator=g).to(dtype) for c in ctx_lens]
    for b, v in enumerate(vecs):
        for j in range(v.shape[0]):
            pages[perm[b, j // page_size], j % page_size] = v[j]
    n = sum(q_lens)
    qh = 5 + p
    qlat = torch.randn(heads, n, r, generator=g).to(dtype)
    q = torch.randn(n, heads * qh, generator=g).to(dtype)
    positions, row_of = [], []
    for b, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        positions += list(range(c - ql, c))
        row_of += [b] * ql
    return dict(qlat=qlat, q=q, pages=pages, bt=perm.to(torch.int32), positions=positions, row_of=row_of,
                vecs=vecs, qh=qh)


def _latent_dense(case, heads, r, p, scale):
    out = torch.zeros(heads, len(case["positions"]), r, dtype=torch.float64)
    for t, (pos, b) in enumerate(zip(case["positions"], case["row_of"])):
        vec = case["vecs"][b][:pos + 1].double()
        qrot = case["q"][t].double().view(heads, case["qh"])[:, 5:5 + p]
        full = torch.cat((case["qlat"][:, t].double(), qrot), -1)
        w = torch.softmax(full @ vec.T * scale, -1)
        out[:, t] = w @ vec[:, :r]
    return out


def _run_latent(case, heads, r, p, scale, splits=1, kernel="auto"):
    K = _K()
    qlat = case["qlat"].to(DEV)
    out = torch.empty_like(qlat)
    scratch = None
    if splits > 1:
        scratch = torch.empty(K.latent_attention_scratch_bytes(qlat.shape[1], heads, r, splits) // 4, device=DEV)
    K.latent_attention(qlat, case["q"].to(DEV), 5, case["qh"], case["pages"].to(DEV), case["bt"].to(DEV),
                       _i32(case["positions"]), _i32(case["row_of"]), out, heads, r, p, scale, splits=splits,
                       scratch=scratch, kernel=kernel)
    return out.cpu().double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("heads,r,p", [(3, 24, 8), (1, 40, 6), (10, 160, 2), (6, 96, 16), (5, 320, 0), (2, 16, 64),
                                       (16, 512, 64), (20, 128, 16), (1, 32, 16), (4, 256, 16)])
def test_latent_attention_kernel_against_dense(dtype, heads, r, p):
    """Both kernels: the generic one (every geometry, both types) and the tensor-core one, which
    bfloat16 takes where the sizes allow (here the last five geometries, (6, 96, 16) and (5, 320, 0)), with four
    warps or, for long latents, eight."""
    scale = 0.3 / math.sqrt(r + p)
    case = _latent_case(r + heads, dtype, heads, r, p, ctx_lens=[70, 1, 33, 200], q_lens=[70, 1, 2, 1], page_size=16)
    want = _latent_dense(case, heads, r, p, scale)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    kernels = ("auto", "generic") if dtype == torch.bfloat16 else ("auto",)
    for kernel in kernels:
        got = _run_latent(case, heads, r, p, scale, kernel=kernel)
        assert (got - want).abs().max() <= tol * want.abs().max(), kernel
    dec = _latent_case(7, dtype, heads, r, p, ctx_lens=[700, 130, 1, 64], q_lens=[1, 1, 1, 1], page_size=8)
    want = _latent_dense(dec, heads, r, p, scale)
    for kernel in kernels:
        for splits in (1, 3, 8):
            got = _run_latent(dec, heads, r, p, scale, splits, kernel=kernel)
            assert (got - want).abs().max() <= tol * want.abs().max(), (kernel, splits)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_latent_attention_finds_a_planted_key(dtype):
    """One key's latent is a large multiple of a direction u, and so is every query: that key takes
    all the weight wherever it is visible, and none where it lies one past the causal edge."""
    heads, r, p, ps = 4, 32, 16, 16  # (bfloat16 runs this geometry on the tensor-core kernel)
    scale = 1.0
    for ctx, q_len, splits in ((600, 1, 1), (600, 1, 5), (600, 40, 1), (48, 48, 1), (130, 3, 2)):
        first_q = ctx - q_len
        spots = [0, 1, ps - 1, ps, ps + 1, first_q - 1, first_q, ctx - 1, 3 * ps - 1, 3 * ps]
        for planted in sorted({s for s in spots if 0 <= s < ctx}):
            case = _latent_case(planted, dtype, heads, r, p, [ctx], [q_len], ps)
            u = torch.zeros(r + p)
            u[3] = 1.0
            for vec_src in (case["vecs"][0],):
                vec_src.mul_(0.05)
                vec_src[planted] = (40 * u).to(dtype)
            page, slot = case["bt"][0, planted // ps], planted % ps
            for j in range(ctx):
                case["pages"][case["bt"][0, j // ps], j % ps] = case["vecs"][0][j]
            case["qlat"][:] = (2 * u[:r]).to(dtype)
            case["q"].zero_()
            got = _run_latent(case, heads, r, p, scale, splits)
            for t, pos in enumerate(case["positions"]):
                hit = got[:, t, 3]
                if pos >= planted:
                    assert (hit - 40).abs().max() < 0.5, (ctx, q_len, planted, pos)
                else:
                    assert hit.abs().max() < 1.0, (ctx, q_len, planted, pos)
            assert page >= 0 and slot >= 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("n,experts,top,ff,width", [(1, 4, 1, 16, 64), (37, 5, 2, 24, 48), (300, 3, 3, 8, 40),
                                                    (130, 10, 3, 88, 264), (20, 3, 2, 12, 36), (700, 6, 2, 200, 136),
                                                    (900, 8, 2, 256, 192), (1500, 5, 3, 128, 64)])
def test_routed_experts_against_plain(dtype, n, experts, top, ff, width):
    from emberserve_b200.parts.base import StepContext
    from emberserve_b200.parts.moe import RoutedGLU, RoutedGLUSpec

    g = torch.Generator().manual_seed(n)
    names = tuple((f"e{e}.gate", f"e{e}.up", f"e{e}.down") for e in range(experts))
    part = RoutedGLU(RoutedGLUSpec(width, ff, experts, top, "router", names), "ffn")
    w = {"router": torch.randn(experts, width, generator=g) * 2}
    for e in range(experts):
        w[f"e{e}.gate"] = torch.randn(ff, width, generator=g) / math.sqrt(width)
        w[f"e{e}.up"] = torch.randn(ff, width, generator=g) / math.sqrt(width)
        w[f"e{e}.down"] = torch.randn(width, ff, generator=g) / math.sqrt(ff)
    w = {k: v.to(dtype) for k, v in w.items()}
    params = {}
    for local, spec in part.param_specs().items():
        t = torch.empty(spec.shape, dtype=dtype, device=DEV)
        for src in spec.sources:
            (t if src.rows is None else t[src.rows[0]:src.rows[1]]).copy_(w[src.name])
        params[local] = t
    part.bind(params)
    x = torch.randn(n, width, generator=g).to(dtype)
    bufs = {}

    def scratch(name, shape, dt):
        bufs[name] = torch.empty(shape, dtype=dt, device=DEV)
        return bufs[name]

    ctx = StepContext(num_tokens=n, num_rows=1, dtype=dtype, device=torch.device(DEV), tokens=None, positions=None,
                      row_of_token=None, cu_q=None, starts=None, q_lens=[n], start_list=[0], scratch=scratch)
    got = part.forward(x.to(DEV), ctx).cpu().double()
    _K().check_status()  # (the last two shapes take the tcgen05 grouped product in bfloat16)
    want = plain.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, experts, top)
    err = (got - want).abs().amax(-1) / want.abs().max()
    if dtype == torch.float32:
        assert err.max() < 2e-5
    else:  # a token whose two candidates lie within bfloat16 rounding may take the other expert
        assert (err > 3e-2).float().mean() <= 0.02
    # each token alone gives what it gave in the batch: rows do not see each other
    if n > 1:
        one = part.forward(x[5:6].to(DEV).contiguous(), StepContext(
            num_tokens=1, num_rows=1, dtype=dtype, device=torch.device(DEV), tokens=None, positions=None,
            row_of_token=None, cu_q=None, starts=None, q_lens=[1], start_list=[0], scratch=scratch)).cpu().double()
        assert (one[0] - got[5]).abs().max() <= 1e-6 * want.abs().max() + (0 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("n,experts,top", [(5, 3, 3), (70, 40, 5), (900, 64, 6), (33, 300, 4), (600, 9, 1)])
def test_routing_alone(n, experts, top):
    """Scores, choice (ties to the lower index), weights with and without renormalisation, and the
    sorted layout: every pair appears once, among the rows of its expert."""
    K = _K()
    g = torch.Generator().manual_seed(n)
    logits = torch.randn(n, experts, generator=g) * 3
    logits[0, :] = 1.5  # all equal: the first `top` experts win
    if experts > 4:
        logits[1, 2] = logits[1, 4] = 9.0  # two equal maxima
    tile = K.moe_tile_rows()
    max_tiles = K.moe_max_tiles(n * top, experts, tile)
    for renorm in (False, True):
        ids = torch.empty(n * top, dtype=torch.int32, device=DEV)
        wts = torch.empty(n * top, device=DEV)
        offsets = torch.empty(3 * experts + 1, dtype=torch.int32, device=DEV)
        perm = torch.full((n * top,), -1, dtype=torch.int32, device=DEV)
        plan = torch.empty(1 + 3 * max_tiles, dtype=torch.int32, device=DEV)
        K.moe_route(logits.to(DEV), top, renorm, ids, wts, offsets, perm, plan, max_tiles)
        s = torch.softmax(logits.double(), -1)
        order = torch.argsort(-logits.double(), dim=-1, stable=True)[:, :top]
        assert torch.equal(ids.cpu().view(n, top).long(), order)
        want = torch.gather(s, 1, order)
        if renorm:
            want = want / want.sum(-1, keepdim=True)
        assert (wts.cpu().view(n, top).double() - want).abs().max() < 1e-6
        off = offsets.cpu()[:experts + 1].tolist()
        assert off[0] == 0 and off[-1] == n * top
        p = perm.cpu().long()
        assert sorted(p.tolist()) == list(range(n * top))
        flat = ids.cpu().long()
        for e in range(experts):
            assert bool((flat[p[off[e]:off[e + 1]]] == e).all())
        pl = plan.cpu().tolist()
        covered = sum(pl[3 + 3 * i] for i in range(pl[0]))
        assert covered == n * top and all(pl[3 + 3 * i] <= tile for i in range(pl[0]))


def test_routing_laid_out_for_tiles_of_256_rows():
    """The layout of prompt steps: every expert's rows start at a multiple of 256, the rows between
    belong to nobody (-1), and every group of 256 rows names its expert or -1."""
    K = _K()
    n, experts, top, align = 1000, 7, 2, K.MOE_BIG_TILE_ROWS
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(n, experts, generator=g) * 2
    logits[:, 3] = -50.0  # an expert that nobody chooses
    max_tiles = K.moe_max_tiles(n * top, experts, K.moe_tile_rows())
    big = torch.empty(K.moe_max_tiles(n * top, experts, align), dtype=torch.int32, device=DEV)
    ids = torch.empty(n * top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n * top, device=DEV)
    offsets = torch.empty(3 * experts + 1, dtype=torch.int32, device=DEV)
    perm = torch.empty(big.numel() * align, dtype=torch.int32, device=DEV)
    plan = torch.empty(1 + 3 * max_tiles, dtype=torch.int32, device=DEV)
    K.moe_route(logits.to(DEV), top, False, ids, wts, offsets, perm, plan, max_tiles, align=align, big=big)
    off, p, flat, b = offsets.cpu().tolist(), perm.cpu().long(), ids.cpu().long(), big.cpu().tolist()
    counts = torch.bincount(flat, minlength=experts).tolist()
    assert counts[3] == 0
    used = []
    for e in range(experts):
        assert off[e] % align == 0
        rows = p[off[e]:off[e] + counts[e]]
        assert bool((rows >= 0).all()) and bool((flat[rows] == e).all())
        used += [e] * (-(-counts[e] // align))
        end = off[e] + (-(-counts[e] // align)) * align
        assert bool((p[off[e] + counts[e]:end] == -1).all())
    assert b[:len(used)] == used and all(x == -1 for x in b[len(used):])
    assert sorted(p[p >= 0].tolist()) == list(range(n * top))
    pl = plan.cpu().tolist()
    assert sum(pl[3 + 3 * i] for i in range(pl[0])) == n * top
    for i in range(pl[0]):
        e, row0, rows = pl[1 + 3 * i], pl[2 + 3 * i], pl[3 + 3 * i]
        assert off[e] <= row0 and row0 + rows <= off[e] + counts[e]


@pytest.mark.parametrize("act", ["relu", "silu", "gelu_tanh"])
def test_gated_activations(act):
    K = _K()
    g = torch.Generator().manual_seed(1)
    gu = torch.randn(5, 2 * 37, generator=g) * 3
    out = torch.empty(5, 37, device=DEV)
    K.glu_act(gu.to(DEV), out, act)
    z = gu[:, :37].double()
    f = {"relu": torch.relu(z), "silu": z * torch.sigmoid(z),
         "gelu_tanh": 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[act]
    assert (out.cpu().double() - f * gu[:, 37:].double()).abs().max() < 1e-5


def test_stream_inject():
    K = _K()
    g = torch.Generator().manual_seed(2)
    emb, tab = torch.randn(11, 20, generator=g).to(torch.bfloat16), torch.randn(3, 20, generator=g).to(torch.bfloat16)
    res = torch.randn(4, 20, generator=g)
    toks = [7, 0, 10, 3]
    for use_emb, row in ((True, 2), (False, 1), (True, None)):
        r = res.to(DEV).clone()
        K.stream_inject(r, _i32(toks), emb.to(DEV) if use_emb else None, tab.to(DEV) if row is not None else None,
                        row or 0)
        want = res.clone()
        if use_emb:
            want += emb[toks].float()
        if row is not None:
            want += tab[row].float()
        assert (r.cpu() - want).abs().max() < 1e-6


# ---- the engine -------------------------------------------------------------------------------

def _oracle(model_dir, reqs):
    cfg, w = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, w, toks, torch.float64).numpy() for rid, toks in reqs}


def _replay(model_dir, name, dtype, steps, slots=4, page_size=None):
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner

    ps = page_size or td.PAGE_SIZES[name]
    pages = TraceReplayer.pages_for(rc.max_live_tokens(steps), ps)
    runner = ModelRunner.from_dir(model_dir, dtype, page_size=ps, num_pages=pages, num_state_slots=slots)
    rp = TraceReplayer(runner)
    outs = {}
    for s in steps:
        o = rp.run_step(s)
        if o is not None:
            outs[s["step"]] = o
        runner.cache.check()
    st = runner.cache.stats()
    assert st.num_sequences == 0 and st.num_free == st.num_pages and st.free_state_slots == st.num_state_slots
    return rc.collect(steps, outs)


def _compare(got, want, reqs, scale, dtype, what):
    errs = np.array([float(np.abs(got[(rid, p)] - want[rid][p]).max()) for rid, toks in reqs
                     for p in range(len(toks))]) / scale
    if dtype == torch.float32:
        assert errs.max() <= TOL32, f"{what}: max |dlogit| / scale {errs.max():.3e}"
    else:
        # bfloat16 against the 64-bit oracle, with weights drawn wide: rounding moves router logits,
        # and where two experts lie that close a token takes the other one (with one expert of four
        # chosen, a few per cent of the positions); a fault moves most positions by far more
        assert np.mean(errs > TOL16) <= 0.10 and np.median(errs) <= TOL16 / 4, (
            f"{what}: {np.mean(errs > TOL16):.3f} of positions over, median {np.median(errs):.3e}")


@pytest.fixture(scope="module")
def cases(dam_dirs):
    out = {}
    for name in td.ALL:
        reqs = rc.make_requests(td.ALL[name]["vocab"], LENGTHS[name], seed=7)
        want = _oracle(dam_dirs[name], reqs)
        out[name] = (reqs, want, max(float(np.abs(v).max()) for v in want.values()))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["dam_a", "dam_b", "dam_c"])
def test_cut_equals_plain(dam_dirs, cases, name, cut, dtype):
    reqs, want, scale = cases[name]
    steps = {"whole": rc.whole, "tail": lambda r: rc.bulk_then_tail(r, 40), "portions": rc.portions,
             "mixed": lambda r: rc.mixed(r, seed=3)}[cut](reqs)
    if cut == "mixed":
        assert rc.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for _, t in reqs)
    got = _replay(dam_dirs[name], name, dtype, steps)
    assert len(got) == sum(len(t) for _, t in reqs)
    _compare(got, want, reqs, scale, dtype, f"{name} {cut}")


def test_batches_of_unequal_requests_equal_each_alone(dam_dirs, cases):
    """In 32 bits a request's logits in a mixed batch, through three state slots and a small pool
    that seven requests share in turn, are those it has alone."""
    name = "dam_b"
    reqs, want, scale = cases[name]
    alone = _replay(dam_dirs[name], name, torch.float32, rc.whole(reqs))
    mixed = _replay(dam_dirs[name], name, torch.float32, rc.mixed(reqs, max_live=3, seed=9), slots=3)
    worst = max(float(np.abs(alone[k] - mixed[k]).max()) for k in alone)
    assert worst <= TOL32 * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_long_decoding_token_by_token(dam_dirs, dtype):
    """A whole request one token per step, from the first token on (the first tokens of a sequence
    see a convolution state of zeros and a one-key softmax), across many pages."""
    name = "dam_a"
    reqs = rc.make_requests(td.ALL[name]["vocab"], [150], seed=21)
    want = _oracle(dam_dirs[name], reqs)
    scale = float(np.abs(want["r0"]).max())
    got = _replay(dam_dirs[name], name, dtype, rc.bulk_then_tail(reqs, 150))
    _compare(got, want, reqs, scale, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dam_dirs, cases, tmp_path, dtype):
    name = "dam_a"
    reqs, want, scale = cases[name]
    steps = rc.mixed(reqs, seed=4)
    out_dir = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(dam_dirs[name]), "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(rc.max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = td.ALL[name]["vocab"]
    outs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
            for s in steps if any(e["want"] for e in s["entries"])}
    _compare(rc.collect(steps, outs), want, reqs, scale, torch.float32 if dtype == "float32" else torch.bfloat16,
             "trace_run")


def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(plain.forward(cfg, w, toks, torch.float64)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["dam_a", "dam_b", "dam_c"])
def test_greedy_generation_through_the_entry_point(dam_dirs, name):
    from emberserve_b200 import LLM, SamplingParams

    cfg, w = plain.read_model_dir(dam_dirs[name])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 5, 11, 30)]
    want = [_plain_greedy(cfg, w, p, 10) for p in prompts]
    for how in (dict(), dict(max_num_batched_tokens=7), dict(enable_cuda_graphs=False, async_scheduling=False)):
        llm = LLM(str(dam_dirs[name]), dtype="float32", device=DEV, block_size=td.PAGE_SIZES[name],
                  num_gpu_blocks=256, max_model_len=128, max_num_seqs=3, **how)
        got = [r.output_token_ids for r in llm.generate(prompts, SamplingParams.greedy(10, ignore_eos=True))]
        assert got == want, how
        st = llm.engine.runner.cache.stats()
        assert st.num_free == st.num_pages and st.free_state_slots == st.num_state_slots


def test_command_line_random_weights_then_generate(tmp_path):
    """`random-weights` writes a Damolorn folder from its config.json; `generate` on it prints the
    tokens that LLM.generate returns (sampled with a seed, bfloat16)."""
    from emberserve_b200 import LLM, SamplingParams

    (tmp_path / "config.json").write_text(json.dumps(td.DAM_A))
    model = tmp_path / "model"
    proc = subprocess.run([sys.executable, "-m", "emberserve_b200", "random-weights", "--config",
                           str(tmp_path / "config.json"), "--out", str(model), "--seed", "5", "--std", "0.3"],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-1500:]
    prompt = [7, 50, 33, 90, 9]
    llm = LLM(str(model), dtype="bfloat16", device=DEV, block_size=16, num_gpu_blocks=64, max_model_len=200)
    want = llm.generate([prompt], SamplingParams(max_tokens=6, temperature=0.7, top_k=20, seed=11))[0]
    proc = subprocess.run(
        [sys.executable, "-m", "emberserve_b200", "generate", "--model", str(model), "--dtype", "bfloat16",
         "--block-size", "16", "--num-blocks", "64", "--max-model-len", "200", "--prompt-ids",
         ",".join(map(str, prompt)), "--max-tokens", "6", "--temperature", "0.7", "--top-k", "20", "--seed", "11"],
        capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-1500:]
    assert [int(t) for t in proc.stdout.split()] == want.output_token_ids


def test_long_prompt_steps_take_the_grouped_tensor_core_products(tmp_path):
    """A prompt of 700 tokens in one step (more than 512 tokens: the experts' products run in their
    tcgen05 grouped form, rows laid out in tiles of 256) gives the logits of the same prompt in
    portions of 200 (the mma.sync kernels), and both follow the 64-bit oracle as closely as bfloat16
    allows.  Experts of 128 x 64 are the smallest the grouped form takes."""
    cfg = json.loads(json.dumps(td.DAM_B))
    cfg["max_positions"] = 1024
    cfg["layers"][0]["mlp"] = {"kind": "moe", "expert": {"ff": 128}, "router": {"experts": 6, "top": 2}}
    cfg["layers"][1]["mlp"] = {"kind": "moe", "expert": {"ff": 256}, "router": {"experts": 3, "top": 3}}
    # (a latent of 256 numbers: the attention kernel with eight warps)
    cfg["layers"][1]["mixer"] = td._mixer(5, 4, 16, 16, 8, 256, 28, 200000.0)
    model = td.write_model(cfg, tmp_path / "m", seed=31)
    reqs = rc.make_requests(cfg["vocab"], [700], seed=2)
    want = _oracle(model, reqs)
    scale = float(np.abs(want["r0"]).max())
    whole = _replay(model, "dam_b", torch.bfloat16, rc.whole(reqs))
    parts = _replay(model, "dam_b", torch.bfloat16, rc.portions(reqs, sizes=(200, 1, 150, 3, 190)))
    _K().check_status()
    _compare(whole, want, reqs, scale, torch.bfloat16, "one step")
    _compare(parts, want, reqs, scale, torch.bfloat16, "portions")
    errs = np.array([float(np.abs(whole[k] - parts[k]).max()) for k in whole]) / scale
    assert np.median(errs) <= TOL16 / 4 and np.mean(errs > TOL16) <= 0.10
