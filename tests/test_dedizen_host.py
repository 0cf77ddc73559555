"""Dedizen through the package's own configuration, loader, cache manager, step function and
replay driver on the CPU (the kernels replaced by their restatements), against the plain
implementation: every way of cutting the same requests gives the plain logits."""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import kernel_refs
import plain_dedizen as plain
import replay_cases as rc
import tiny_dedizen as td
from host_harness import host_runner

from emberserve_b200.config.dedizen import DedizenConfig
from emberserve_b200.config.model import ConfigError
from emberserve_b200.engine.replay import TraceReplayer
from emberserve_b200.parts.base import FixedState, PagedKV
from emberserve_b200.registry import build_decoder, load_config

LENGTHS = {"ded_a": [1, 2, 9, 23, 40, 31], "ded_b": [3, 17, 50, 8, 70, 33], "ded_c": [2, 48, 11, 61, 35, 5]}


@pytest.fixture(autouse=True)
def _refs(monkeypatch):
    kernel_refs.install(monkeypatch)


@pytest.fixture(scope="module")
def ded_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("dedizen")
    return {name: td.write_model(cfg, root / name, td.SEEDS[name]) for name, cfg in td.ALL.items()}


def _replay(model_dir, name, steps, slots=4):
    ps = td.PAGE_SIZES[name]
    runner = host_runner(model_dir, page_size=ps, num_pages=TraceReplayer.pages_for(rc.max_live_tokens(steps), ps),
                         num_state_slots=slots)
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


def _oracle(model_dir, reqs):
    cfg, w = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, w, toks, torch.float64).numpy() for rid, toks in reqs}


@pytest.mark.parametrize("name", ["ded_a", "ded_b", "ded_c"])
def test_all_cuts_equal_plain(ded_dirs, name):
    reqs = rc.make_requests(td.ALL[name]["vocab"], LENGTHS[name], seed=7)
    want = _oracle(ded_dirs[name], reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    cuts = {"whole": rc.whole(reqs), "tail": rc.bulk_then_tail(reqs, 12), "portions": rc.portions(reqs),
            "mixed": rc.mixed(reqs, seed=3)}
    for cut, steps in cuts.items():
        got = _replay(ded_dirs[name], name, steps)
        worst = max(float(np.abs(got[(rid, p)] - want[rid][p]).max()) for rid, toks in reqs for p in range(len(toks)))
        assert worst <= 5e-5 * scale, f"{name} {cut}: max |dlogit| {worst:.3e} (scale {scale:.3f})"


def test_mixed_reuses_pages_and_state_slots(ded_dirs):
    name = "ded_b"
    reqs = rc.make_requests(td.ALL[name]["vocab"], [40, 33, 70, 21, 64, 18, 50], seed=11)
    steps = rc.mixed(reqs, max_live=3, seed=5)
    assert rc.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for _, t in reqs)
    got = _replay(ded_dirs[name], name, steps, slots=3)  # seven requests through three slots
    want = _oracle(ded_dirs[name], reqs)
    for rid, toks in reqs:
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[rid][p]).max() < 1e-3


def test_pages_of_finished_chunks_go_back_while_the_request_lives(ded_dirs):
    """A chunk mask of 5 positions over pages of 4: after 23 tokens only the pages that hold
    positions 20.. are still held by the attention's group."""
    from emberserve_b200.engine.runner import StepRow

    runner = host_runner(ded_dirs["ded_a"], page_size=4, num_pages=16, num_state_slots=2)
    toks = list(range(1, 24))
    runner.cache.admit(0, len(toks))
    runner.step([StepRow(0, toks, 0, [len(toks) - 1])])
    table = runner.cache.table(0, 0)
    assert [p >= 0 for p in table] == [False] * 5 + [True]
    runner.cache.check()
    runner.cache.extend(0, 26)
    out = runner.step([StepRow(0, [5, 6, 7], 23, [0, 1, 2])])  # crosses the chunk border at 25
    cfg, w = plain.read_model_dir(ded_dirs["ded_a"])
    want = plain.forward(cfg, w, toks + [5, 6, 7], torch.float64)[-3:]
    assert (out.double() - want).abs().max() < 1e-4 * want.abs().max()
    runner.cache.release(0)
    runner.cache.check()


def test_config_round_trip(tmp_path):
    for cfg in td.ALL.values():
        typed = DedizenConfig.from_dict(cfg)
        assert DedizenConfig.from_dict(json.loads(json.dumps(typed.to_dict()))) == typed
    typed = td.typed(td.DED_B)
    typed.save(tmp_path)
    assert load_config(tmp_path) == typed
    assert typed.layers[1].mixer.left.rot_scaling is None and typed.layers[3].mixer.left.rot_scaling.factor == 8.0
    assert td.typed(td.DED_C).layers[0].mixer.left.rot_dims == 0


def test_config_refusals():
    def broken(change):
        bad = json.loads(json.dumps(td.DED_A))
        change(bad)
        with pytest.raises(ConfigError):
            DedizenConfig.from_dict(bad)

    broken(lambda c: c["layers"][0].update(type="something_else"))
    broken(lambda c: c["layers"][0]["mixer"].update(blocks=5))  # 36 channels in 5 blocks
    broken(lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4))  # 6 heads over 4
    broken(lambda c: c["layers"][1]["mixer"]["left"].update(vdim=12))  # the values are the keys
    broken(lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]))
    broken(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=10))
    broken(lambda c: c["layers"][2]["mixer"].pop("gate_cap"))
    broken(lambda c: c["layers"][2]["mlp"].update(kind="moe"))
    broken(lambda c: c.pop("norm"))


def test_parameter_table_names_every_checkpoint_tensor():
    for cfg in td.ALL.values():
        dec = build_decoder(td.typed(cfg))
        named = {src.name: None for spec in dec.param_table().values() for src in spec.sources}
        assert set(named) == set(td.tensor_shapes(cfg))


def test_cache_entries_per_layer():
    dec = build_decoder(td.typed(td.DED_B))
    entries = dec.cache_entries()
    # mLSTM: one state; parallel: pages + memory; RG-LRU with one tap: its state alone; parallel
    assert [type(e) for e in entries] == [FixedState, PagedKV, FixedState, FixedState, PagedKV, FixedState]
    assert entries[1] == PagedKV(4, 16, None, 16) and entries[4] == PagedKV(1, 24, None, 400)
    assert entries[0].shape == (1, 20 * 28 + 20 + 1) and entries[3].shape == (40,)
    dec = build_decoder(td.typed(td.DED_C))
    assert [call.cache for call in dec.spec.order] == [(0, 1), 2, (3, 4), (5, 6)]
    assert dec.cache_entries()[3] == FixedState((4, 130), "float32")  # five taps keep four inputs


def test_random_weights_folder_loads_and_steps(tmp_path):
    """The random-weights mode writes every tensor the design names, and the folder loads through
    the registry and runs a step; the gate rows that pad the attention's fused projection are zero."""
    from emberserve_b200.engine.runner import StepRow
    from emberserve_b200.weights.loader import write_random_model

    cfg = td.typed(td.DED_A)
    out = write_random_model(cfg, tmp_path / "m", seed=3, std=0.2)
    _, w = plain.read_model_dir(out)
    assert set(w) == set(td.tensor_shapes(td.DED_A))
    runner = host_runner(out, page_size=8, num_pages=8, num_state_slots=2)
    attn = runner.decoder.blocks[1].mixer.left
    assert bool((attn.wqkv[attn.gate_at + 6:] == 0).all()) and bool((attn.bqkv[attn.gate_at:] == 0).all())
    runner.cache.admit(0, 7)
    logits = runner.step([StepRow(0, [1, 2, 3, 4, 5, 6, 7], 0, [6])])
    want = plain.forward(td.DED_A, w, [1, 2, 3, 4, 5, 6, 7], torch.float64)[-1]
    assert (logits[0].double() - want).abs().max() < 1e-4 * want.abs().max()
