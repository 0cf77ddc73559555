"""Dedizen on the GPU: every new kernel alone against its restatement and against the plain
implementation (``plain_dedizen``), keys that one score singles out just inside and just outside a
chunk, at page borders, far back and first in a sequence, the sink, memories whose slots change
hands, the engine under every way of cutting the same requests, batches against each request alone,
long decoding, other sizes, and greedy generation through the entry point and its scheduler."""

from __future__ import annotations

import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import kernel_refs as R
import plain_dedizen as plain
import replay_cases as rc
import tiny_dedizen as td

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
LENGTHS = {"ded_a": [1, 2, 9, 23, 40, 31, 130], "ded_b": [3, 17, 50, 8, 70, 33, 150],
           "ded_c": [2, 48, 11, 61, 35, 5, 97]}
TOL32 = 5e-5  # of the largest |logit|
TOL16 = 6e-2  # bfloat16 against the 64-bit plain implementation, weights drawn wide
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _K():
    from emberserve_b200 import kernels

    return kernels


def _close(got, want, dtype, what=""):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    scale = float(want.abs().max()) + 1e-30
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    err = float((got - want).abs().max()) / scale
    assert err <= tol, f"{what}: {err:.3e} of scale {scale:.3e}"


@pytest.fixture(scope="module")
def ded_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("dedizen")
    return {name: td.write_model(cfg, root / name, td.SEEDS[name]) for name, cfg in td.ALL.items()}


# ---- kernels alone ----------------------------------------------------------------------------

@DTYPES
@pytest.mark.parametrize("act", ["relu", "relu2", "gelu_tanh", "silu"])
def test_ungated_activations(dtype, act):
    g = torch.Generator().manual_seed(1)
    x = (3 * torch.randn(37, 50, generator=g)).to(dtype)
    want = torch.empty_like(x)
    R.unary_act(x, want, act)
    got = torch.empty_like(x, device=DEV)
    _K().unary_act(x.to(DEV), got, act)
    _close(got, want, dtype, act)
    if act == "relu2":  # against the definition itself
        assert torch.equal(want.float(), (torch.relu(x.float()) ** 2).to(dtype).float())


@DTYPES
@pytest.mark.parametrize("taps,identity,bias", [(1, False, True), (2, False, True), (5, False, False), (3, True, True)])
def test_convolution_with_bias_on_a_column_range_through_slots_that_change_hands(dtype, taps, identity, bias):
    g = torch.Generator().manual_seed(taps)
    c, pad = 22, 10
    w = (0.7 * torch.randn(c, taps, generator=g)).to(dtype)
    bb = torch.randn(c, generator=g).to(dtype) if bias else None
    state_ref = torch.randn(3, max(taps - 1, 1), c, generator=g)[:, :taps - 1]  # stale contents
    state = state_ref.clone().to(DEV)
    # three requests in portions of 1..5 tokens through two slots; slot 1 is handed on and zeroed
    plan = [([0, 1], [3, 1]), ([0, 1], [1, 1]), ([0, 1], [2, 5]), ([2, 0], [4, 1])]
    slot_of = {0: 0, 1: 1, 2: 1}
    for s in (0, 1):
        state_ref[s] = 0
        state[s] = 0
    for step, (reqs, lens) in enumerate(plan):
        if step == 3:
            state_ref[1] = 0
            state[1] = 0
        n = sum(lens)
        wide = torch.randn(n, pad + c, generator=g).to(dtype)
        cu = _i32(np.concatenate([[0], np.cumsum(lens)]))
        row_of = _i32(np.repeat(np.arange(len(lens)), lens))
        slots = _i32([slot_of[r] for r in reqs])
        want = torch.empty(n, c, dtype=dtype)
        R.causal_taps(wide[:, pad:], w, state_ref if taps > 1 else None, slots.cpu(), cu.cpu(), row_of.cpu(), want,
                      len(lens), bias=bb, identity=identity)
        got = torch.empty(n, c, dtype=dtype, device=DEV)
        _K().causal_taps(wide.to(DEV)[:, pad:], w.to(DEV), state if taps > 1 else None, slots, cu, row_of, got,
                         len(lens), bias=None if bb is None else bb.to(DEV), identity=identity)
        _close(got, want, dtype, f"step {step}")
    if taps > 1:
        _close(state, state_ref, torch.float32, "state")


def _paged(g, dtype, nkv, d, page_size, ctx_lens):
    """Block tables over shuffled pages for requests of the given lengths."""
    pages_per = [-(-c // page_size) for c in ctx_lens]
    total = sum(pages_per) + 3
    perm = torch.randperm(total, generator=g).tolist()
    bt = torch.zeros(len(ctx_lens), max(pages_per), dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    kc = torch.randn(total, nkv, page_size, d, generator=g).to(dtype)  # stale contents everywhere
    vc = torch.randn(total, nkv, page_size, d, generator=g).to(dtype)
    return bt, kc, vc


@DTYPES
@pytest.mark.parametrize("pairing,rot,d,normed,vk", [("interleaved", 4, 8, True, True), ("interleaved", 16, 16, True, False),
                                                      ("half", 6, 24, False, True), ("interleaved", 0, 40, True, True)])
def test_rotation_norm_and_cache_write(dtype, pairing, rot, d, normed, vk):
    g = torch.Generator().manual_seed(rot + d)
    nh, nkv, ps = 6, 2, 4
    starts, qlens = [0, 9, 3], [7, 1, 5]
    bt, kc, vc = _paged(g, dtype, nkv, d, ps, [s + q for s, q in zip(starts, qlens)])
    n = sum(qlens)
    cols = (nh + nkv * (1 if vk else 2)) * d + 8
    proj = torch.randn(n, cols, generator=g).to(dtype)
    pos = _i32(np.concatenate([np.arange(s, s + q) for s, q in zip(starts, qlens)]))
    row_of = _i32(np.repeat(np.arange(3), qlens))
    table = None
    if rot:
        inv = (50.0 ** (-torch.arange(0, rot, 2, dtype=torch.float32) / rot))
        table = R.rope_table(inv, 32) * 1.3
    eps = 1e-5 if normed else None
    want = (proj.clone(), kc.clone(), vc.clone())
    R.qk_prep(want[0], nh, nkv, d, pos.cpu(), row_of.cpu(), table, rot, pairing, eps, want[1], want[2], bt, vk)
    got = (proj.to(DEV), kc.to(DEV), vc.to(DEV))
    _K().qk_prep(got[0], nh, nkv, d, pos, row_of, None if table is None else table.to(DEV), rot, pairing, eps,
                 got[1], got[2], bt.to(DEV), vk)
    for a, b, what in zip(got, want, ("q", "k cache", "v cache")):
        _close(a, b, dtype, what)
    # the oracle's rotation on one head, and the value that is the key as projected
    if rot and pairing == "interleaved" and vk:
        freq = (50.0 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot))
        t = 5  # a token of request 0, position 5
        x = proj[t, :d].double()[None, None, :].repeat(6, 1, 1)
        turned = plain.rotate_interleaved(x, freq, 1.3)[5, 0]
        if normed:
            turned = plain.rms(turned, 1e-5)
        _close(got[0][t, :d], turned, dtype, "against the plain rotation")
        page, slot = int(bt[0, 5 // ps]), 5 % ps
        assert torch.equal(got[2][page, 0, slot].cpu(), proj[t, nh * d:nh * d + d])


def _attention_case(g, dtype, nh, nkv, d, ps, starts, qlens):
    ctx = [s + q for s, q in zip(starts, qlens)]
    bt, kc, vc = _paged(g, dtype, nkv, d, ps, ctx)
    n = sum(qlens)
    q = torch.randn(n, nh * d + 16, generator=g).to(dtype)
    gate = torch.randn(n, nh + 3, generator=g).to(dtype)
    sinks = torch.randn(nh, generator=g)
    cu = _i32(np.concatenate([[0], np.cumsum(qlens)]))
    return q, gate, sinks, bt, kc, vc, cu, _i32(starts), n


def _run_attention(case, nh, nkv, d, scale, max_q, rows, chunk, window, use_sink, use_gate, splits=1, dev=True):
    q, gate, sinks, bt, kc, vc, cu, st, n = case
    mod = _K() if dev else R
    mv = (lambda t: t.to(DEV)) if dev else (lambda t: t.cpu())
    out = torch.zeros(n, nh * d, dtype=q.dtype, device=DEV if dev else "cpu")
    scratch = None
    if splits > 1 and dev:
        scratch = torch.empty(mod.attention_scratch_bytes(n, nh, d, splits) // 4, dtype=torch.float32, device=DEV)
    mod.paged_attention_masked(mv(q), out, mv(kc), mv(vc), mv(bt), mv(cu), mv(st), rows, n, nh, nkv, d, scale, max_q,
                               window=window, chunk=chunk, sinks=mv(sinks) if use_sink else None,
                               gate=mv(gate) if use_gate else None, splits=splits, scratch=scratch)
    return out


@DTYPES
@pytest.mark.parametrize("nh,nkv,d,ps,chunk,window", [(6, 2, 8, 4, 5, None), (4, 4, 16, 16, 16, None), (5, 1, 40, 8, 64, None),
                                                       (2, 1, 24, 16, 7, 4), (8, 8, 64, 16, None, None), (3, 3, 128, 32, 50, None)])
def test_masked_attention_against_dense(dtype, nh, nkv, d, ps, chunk, window):
    g = torch.Generator().manual_seed(nh * d)
    starts, qlens = [0, 61, 17, 130, 5], [33, 1, 20, 1, 2]  # prompts, portions and single tokens in one step
    case = _attention_case(g, dtype, nh, nkv, d, ps, starts, qlens)
    for use_sink, use_gate in ((True, True), (False, True), (True, False), (False, False)):
        want = _run_attention(case, nh, nkv, d, 0.4, max(qlens), 5, chunk, window, use_sink, use_gate, dev=False)
        got = _run_attention(case, nh, nkv, d, 0.4, max(qlens), 5, chunk, window, use_sink, use_gate)
        _close(got, want, dtype, f"sink={use_sink} gate={use_gate}")
    # single tokens only, keys split over blocks and merged
    starts, qlens = [200, 7, 64, 0], [1, 1, 1, 1]
    case = _attention_case(g, dtype, nh, nkv, d, ps, starts, qlens)
    want = _run_attention(case, nh, nkv, d, 0.4, 1, 4, chunk, window, True, True, dev=False)
    for splits in (1, 2, 5):
        got = _run_attention(case, nh, nkv, d, 0.4, 1, 4, chunk, window, True, True, splits=splits)
        _close(got, want, dtype, f"splits={splits}")


@DTYPES
@pytest.mark.parametrize("d", [16, 128], ids=["generic", "tensor-core-size"])
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
def test_a_planted_key_shows_at_chunk_and_page_edges(dtype, decode, d):
    """One key is made to win the softmax (its dot product with one query stands out) and its value
    is a one-hot: the output shows whether the query saw it.  Chunks of 48 over pages of 16: the
    first key of the query's chunk (also the first of a page) is seen, the last key of the chunk
    before is not; a key far back in the same chunk across three pages is; the query itself is."""
    nh, nkv, ps, chunk = 2, 1, 16, 48
    g = torch.Generator().manual_seed(5)
    qpos = 48 * 3 + 40  # position 184, chunk 144..191
    for key, seen in ((144, True), (143, False), (145, True), (160, True), (184, True), (0, False), (96, False)):
        start, qlen = (qpos, 1) if decode else (qpos - 9, 12)
        case = list(_attention_case(g, dtype, nh, nkv, d, ps, [start], [qlen]))
        q, bt, kc, vc = case[0], case[3], case[4].float() * 0.1, case[5].float() * 0.1
        row = qpos - start
        q[row, :nh * d] = 0
        q[row, :d] = 4.0
        q[row, d:2 * d] = 4.0
        page, slot = int(bt[0, key // ps]), key % ps
        kc[page, 0, slot] = 4.0
        vc[page, 0, slot] = 0
        vc[page, 0, slot, 3] = 50.0
        case[4], case[5] = kc.to(dtype), vc.to(dtype)
        out = _run_attention(case, nh, nkv, d, 4.0 / d, qlen, 1, chunk, None, False, False)
        got = float(out[row, 3])
        assert (got > 40.0) == seen, f"key {key} from position {qpos}: {got}"
        want = _run_attention(case, nh, nkv, d, 4.0 / d, qlen, 1, chunk, None, False, False, dev=False)
        _close(out, want, dtype, f"key {key}")


@DTYPES
def test_the_sink_takes_weight_and_has_no_value(dtype):
    """With one key only (the first token of a sequence) the output is v * 1 / (1 + exp(sink - s))."""
    nh, d = 3, 8
    g = torch.Generator().manual_seed(9)
    case = list(_attention_case(g, dtype, nh, nh, d, 4, [0], [1]))
    case[2] = torch.tensor([-30.0, 0.0, 2.0])
    q, bt, kc, vc = case[0], case[3], case[4], case[5]
    out = _run_attention(case, nh, nh, d, 0.5, 1, 1, 7, None, True, False).float().cpu()
    page = int(bt[0, 0])
    for h in range(nh):
        s = float((q[0, h * d:(h + 1) * d].float() * kc[page, h, 0].float()).sum()) * 0.5
        want = vc[page, h, 0].float() / (1 + math.exp(float(case[2][h]) - s))
        assert (out[0, h * d:(h + 1) * d] - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * (
            want.abs().max() + 1e-3)


@DTYPES
def test_mean_of_two_normed_branches(dtype):
    g = torch.Generator().manual_seed(2)
    for c in (40, 250, 2048):
        a, b = (3 * torch.randn(9, c, generator=g)).to(dtype), torch.randn(9, c, generator=g).to(dtype)
        wa, wb = torch.randn(c, generator=g).to(dtype), torch.randn(c, generator=g).to(dtype)
        want = 0.5 * (plain.rms(a.double(), 1e-5) * wa.double() + plain.rms(b.double(), 1e-5) * wb.double())
        got = torch.empty(9, c, dtype=dtype, device=DEV)
        _K().norm_mean2(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-5, got)
        _close(got, want, dtype, f"width {c}")


@DTYPES
@pytest.mark.parametrize("h,d,v,normaliser", [(3, 6, 10, False), (1, 33, 70, False), (4, 9, 65, True), (2, 130, 64, True),
                                               (2, 256, 8, False), (5, 4, 4, True)])
def test_matrix_memory_in_portions_through_slots_with_stale_contents(dtype, h, d, v, normaliser):
    g = torch.Generator().manual_seed(h * d + v)
    per = d * v + (d + 1 if normaliser else 0)
    state_ref = torch.randn(4, h, per, generator=g)
    state_ref[[0, 2]] = 0  # the two slots in use were zeroed when they were handed out
    state = state_ref.clone().to(DEV)
    decay = torch.rand(h, generator=g) * 0.5 + 0.5
    qk, vv, pad = h * d, h * v, 5
    for step, lens in enumerate(([21, 3], [1, 1], [2, 40], [1, 17])):
        n = sum(lens)
        wide = (0.6 * torch.randn(n, pad + 2 * qk + vv, generator=g)).to(dtype)
        cu, slots = _i32(np.concatenate([[0], np.cumsum(lens)])), _i32([2, 0])
        a = torch.rand(n, h, generator=g) * 0.4 + 0.6
        b = torch.rand(n, h, generator=g) + 0.1
        floor = torch.rand(n, h, generator=g) * 0.2
        kw = dict(act="silu", decay_head=decay) if not normaliser else dict(q_scale=d ** -0.5, a=a, b=b, denom_eps=1e-6)
        want, wden = torch.zeros(n, vv), torch.zeros(n, h)
        R.matrix_recurrence(wide[:, pad:pad + qk], wide[:, pad + qk:pad + 2 * qk], wide[:, pad + 2 * qk:], h, d, v,
                            state_ref, slots.cpu(), cu.cpu(), 2, want,
                            **(kw if not normaliser else dict(kw, denom_floor=floor, denom=wden)))
        dw = wide.to(DEV)
        got, gden = torch.zeros(n, vv, device=DEV), torch.zeros(n, h, device=DEV)
        dkw = {k: (x.to(DEV) if isinstance(x, torch.Tensor) else x) for k, x in kw.items()}
        if normaliser:
            dkw.update(denom_floor=floor.to(DEV), denom=gden)
        _K().matrix_recurrence(dw[:, pad:pad + qk], dw[:, pad + qk:pad + 2 * qk], dw[:, pad + 2 * qk:], h, d, v, state,
                               slots, cu, 2, got, **dkw)
        _close(got, want, torch.float32, f"step {step}")
        if normaliser:
            _close(gden, wden, torch.float32, f"denominators of step {step}")
    _close(state[:, :, :d * v + (d if normaliser else 0)], state_ref[:, :, :d * v + (d if normaliser else 0)],
           torch.float32, "state")
    assert torch.equal(state[[1, 3]].cpu(), state_ref[[1, 3]])  # slots of other requests are untouched


def test_lightning_attention_kernel_against_the_plain_recurrence():
    """S_t = decay S + k v^T, o = S^T q through the kernel, against the plain mixer with identity
    projections around it (q, k, v given directly)."""
    g = torch.Generator().manual_seed(4)
    h, d, v, t = 2, 12, 20, 75
    q, k, vv = (torch.randn(t, h * x, generator=g) for x in (d, d, v))
    decay = [0.7, 0.999]
    want = torch.zeros(t, h, v, dtype=torch.float64)
    silu = torch.nn.functional.silu
    for head in range(h):
        S = torch.zeros(d, v, dtype=torch.float64)
        for i in range(t):
            S = decay[head] * S + torch.outer(silu(k[i, head * d:(head + 1) * d].double()), silu(vv[i, head * v:(head + 1) * v].double()))
            want[i, head] = S.T @ silu(q[i, head * d:(head + 1) * d].double())
    state = torch.zeros(1, h, d * v, device=DEV)
    got = torch.zeros(t, h * v, device=DEV)
    _K().matrix_recurrence(q.to(DEV), k.to(DEV), vv.to(DEV), h, d, v, state, _i32([0]), _i32([0, t]), 1, got, act="silu",
                           decay_head=torch.tensor(decay, device=DEV))
    _close(got, want.reshape(t, -1), torch.float32, "lightning")


def test_mlstm_gates_over_many_tokens_and_steps():
    g = torch.Generator().manual_seed(6)
    h = 3
    state_ref = torch.zeros(2, h, 11)
    state = state_ref.clone().to(DEV)
    bi, bf = torch.randn(h, generator=g), 2 + torch.randn(h, generator=g)
    for lens in ([70, 1], [1, 33], [5, 2]):
        n = sum(lens)
        pre = 3 * torch.randn(n, 2 * h, generator=g)
        cu, slots = _i32(np.concatenate([[0], np.cumsum(lens)])), _i32([1, 0])
        want = [torch.zeros(n, h) for _ in range(3)]
        R.mlstm_gates(pre, bi, bf, 4.0, state_ref, 10, slots.cpu(), cu.cpu(), 2, *want)
        got = [torch.zeros(n, h, device=DEV) for _ in range(3)]
        _K().mlstm_gates(pre.to(DEV), bi.to(DEV), bf.to(DEV), 4.0, state, 10, slots, cu, 2, *got)
        for a, b, what in zip(got, want, ("decay", "input scale", "floor")):
            _close(a, b, torch.float32, what)
    _close(state, state_ref, torch.float32, "running maximum")
    assert float(state_ref[:, :, 10].abs().max()) > 0


@DTYPES
@pytest.mark.parametrize("c,groups", [(18, 3), (260, 4), (70, 1), (600, 1), (3000, 2)])
def test_norm_and_gate_behind_a_memory(dtype, c, groups):
    g = torch.Generator().manual_seed(c)
    n = 7
    o = 5 * torch.randn(n, c, generator=g)
    den = torch.rand(n, groups, generator=g) + 0.5
    w = torch.randn(c, generator=g).to(dtype)
    wide = torch.randn(n, c + 6, generator=g).to(dtype)
    for use_den, use_gate in ((True, True), (False, False)):
        x = o.double().view(n, groups, -1) / (den.double()[:, :, None] if use_den else 1.0)
        want = plain.rms(x, 1e-5).reshape(n, c) * w.double()
        if use_gate:
            want = want * torch.sigmoid(wide[:, 6:].double())
        got = torch.empty(n, c, dtype=dtype, device=DEV)
        _K().group_norm_gate(o.to(DEV), groups, 1e-5, w.to(DEV), wide.to(DEV)[:, 6:] if use_gate else None, got,
                             denom=den.to(DEV) if use_den else None)
        _close(got, want, dtype, f"denom={use_den}")


@DTYPES
@pytest.mark.parametrize("c,blocks", [(36, 3), (40, 1), (130, 5), (512, 2)])
def test_gated_diagonal_recurrence_in_portions(dtype, c, blocks):
    g = torch.Generator().manual_seed(c)
    state_ref = torch.randn(3, c, generator=g)
    state_ref[[0, 1]] = 0
    state = state_ref.clone().to(DEV)
    br, bi, lam = (torch.randn(blocks, c // blocks, generator=g).to(dtype), torch.randn(blocks, c // blocks, generator=g).to(dtype),
                   (-2 + torch.randn(c, generator=g)).to(dtype))
    for lens in ([30, 2], [1, 1], [3, 19]):
        n = sum(lens)
        u = torch.randn(n, c, generator=g).to(dtype)
        wide = torch.randn(n, c + 4, generator=g).to(dtype)
        pre = 2 * torch.randn(2, blocks, n, c // blocks, generator=g)
        cu, slots = _i32(np.concatenate([[0], np.cumsum(lens)])), _i32([1, 0])
        want = torch.empty(n, c, dtype=dtype)
        R.rglru_scan(u, pre, br, bi, lam, wide[:, :c], True, 8.0, state_ref, slots.cpu(), cu.cpu(), 2, want, blocks)
        got = torch.empty(n, c, dtype=dtype, device=DEV)
        _K().rglru_scan(u.to(DEV), pre.to(DEV), br.to(DEV), bi.to(DEV), lam.to(DEV), wide.to(DEV)[:, :c], True, 8.0,
                        state, slots, cu, 2, got, blocks)
        _close(got, want, dtype, "out")
    _close(state, state_ref, torch.float32, "state")


# ---- one mechanism per model --------------------------------------------------------------------

ONE_MIXER = {
    "attention": td._parallel(td._left(4, 2, 16, 6, 8, 1000.0, (2.0, 8, 2.0, 0.5)), td._right(1, 4, 4, (0.9,)), None),
    "attention_64": td._parallel(td._left(4, 2, 64, 20, 32, 5000.0, (4.0, 32, 8.0, 1.0)), td._right(1, 4, 4, (0.9,)), None),
    "memory": td._parallel(td._left(1, 1, 8, 2, 0, 0.0), td._right(3, 10, 12, (0.4, 0.9, 0.995)), None),
    "mlstm": td._mlstm(2, 12, 20, 3.0, None),
    "rglru": td._rglru(48, 4, 4, None),
    "feed_forward": td._rglru(8, 1, 1, 100),
}


@DTYPES
@pytest.mark.parametrize("which", sorted(ONE_MIXER))
def test_one_layer_models_in_prompt_and_token_by_token(tmp_path, which, dtype):
    cfg = {"architecture": "Dedizen", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "max_positions": 256,
           "layers": [ONE_MIXER[which]]}
    model = td.write_model(cfg, tmp_path / which, 31)
    reqs = rc.make_requests(50, [45, 90], seed=1)
    want = _oracle(model, reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    for steps in (rc.whole(reqs), rc.bulk_then_tail(reqs, 90)):
        got = _replay(model, None, dtype, steps, page_size=8)
        _compare(got, want, reqs, scale, dtype, which)


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
        assert errs.max() <= TOL16 and np.median(errs) <= TOL16 / 4, (
            f"{what}: max {errs.max():.3e}, median {np.median(errs):.3e}")


@pytest.fixture(scope="module")
def cases(ded_dirs):
    out = {}
    for name in td.ALL:
        reqs = rc.make_requests(td.ALL[name]["vocab"], LENGTHS[name], seed=7)
        want = _oracle(ded_dirs[name], reqs)
        out[name] = (reqs, want, max(float(np.abs(v).max()) for v in want.values()))
    return out


@DTYPES
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["ded_a", "ded_b", "ded_c"])
def test_cut_equals_plain(ded_dirs, cases, name, cut, dtype):
    reqs, want, scale = cases[name]
    steps = {"whole": rc.whole, "tail": lambda r: rc.bulk_then_tail(r, 40), "portions": rc.portions,
             "mixed": lambda r: rc.mixed(r, seed=3)}[cut](reqs)
    if cut == "mixed":
        assert rc.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for _, t in reqs)
    got = _replay(ded_dirs[name], name, dtype, steps)
    assert len(got) == sum(len(t) for _, t in reqs)
    _compare(got, want, reqs, scale, dtype, f"{name} {cut}")


def test_batches_of_unequal_requests_equal_each_alone(ded_dirs, cases):
    """In 32 bits a request's logits in a mixed batch, through three state slots and a small pool
    that seven requests share in turn, are those it has alone."""
    name = "ded_b"
    reqs, want, scale = cases[name]
    alone = _replay(ded_dirs[name], name, torch.float32, rc.whole(reqs))
    mixed = _replay(ded_dirs[name], name, torch.float32, rc.mixed(reqs, max_live=3, seed=9), slots=3)
    worst = max(float(np.abs(alone[k] - mixed[k]).max()) for k in alone)
    assert worst <= TOL32 * scale


@DTYPES
def test_long_decoding_token_by_token(ded_dirs, dtype):
    """A whole request one token per step, from the first token on (zero states, a one-key softmax
    beside its sink), across many pages and chunks."""
    name = "ded_a"
    reqs = rc.make_requests(td.ALL[name]["vocab"], [150], seed=21)
    want = _oracle(ded_dirs[name], reqs)
    scale = float(np.abs(want["r0"]).max())
    got = _replay(ded_dirs[name], name, dtype, rc.bulk_then_tail(reqs, 150))
    _compare(got, want, reqs, scale, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(ded_dirs, cases, tmp_path, dtype):
    name = "ded_c"
    reqs, want, scale = cases[name]
    steps = rc.mixed(reqs, seed=4)
    out_dir = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(ded_dirs[name]), "--dtype", dtype,
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


@pytest.mark.parametrize("name", ["ded_a", "ded_b", "ded_c"])
def test_greedy_generation_through_the_entry_point(ded_dirs, name):
    from emberserve_b200 import LLM, SamplingParams

    cfg, w = plain.read_model_dir(ded_dirs[name])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 5, 11, 30)]
    want = [_plain_greedy(cfg, w, p, 10) for p in prompts]
    for how in (dict(), dict(max_num_batched_tokens=7), dict(enable_cuda_graphs=False, async_scheduling=False)):
        llm = LLM(str(ded_dirs[name]), dtype="float32", device=DEV, block_size=td.PAGE_SIZES[name],
                  num_gpu_blocks=256, max_model_len=128, max_num_seqs=3, **how)
        got = [r.output_token_ids for r in llm.generate(prompts, SamplingParams.greedy(10, ignore_eos=True))]
        assert got == want, how
        st = llm.engine.runner.cache.stats()
        assert st.num_free == st.num_pages and st.free_state_slots == st.num_state_slots


def test_command_line_random_weights_then_generate(tmp_path):
    """`random-weights` writes a Dedizen folder from its config.json; `generate` on it prints the
    tokens that LLM.generate returns (sampled with a seed, bfloat16, decode steps from CUDA graphs)."""
    from emberserve_b200 import LLM, SamplingParams

    (tmp_path / "config.json").write_text(json.dumps(td.DED_B))
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
