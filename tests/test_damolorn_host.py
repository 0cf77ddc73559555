"""Damolorn through the package's own configuration, loader, cache manager, step function and
replay driver on the CPU (the kernels replaced by their restatements), against the plain
implementation: every way of cutting the same requests gives the plain logits."""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import kernel_refs
import plain_damolorn as plain
import replay_cases as rc
import tiny_damolorn as td
from host_harness import host_runner

from emberserve_b200.config.damolorn import DamolornConfig
from emberserve_b200.config.model import ConfigError
from emberserve_b200.engine.replay import TraceReplayer
from emberserve_b200.registry import build_decoder, load_config

LENGTHS = {"dam_a": [1, 2, 9, 23, 40, 31], "dam_b": [3, 17, 50, 8, 70, 33], "dam_c": [2, 48, 11, 61, 35, 5]}


@pytest.fixture(autouse=True)
def _refs(monkeypatch):
    kernel_refs.install(monkeypatch)


@pytest.fixture(scope="module")
def dam_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("damolorn")
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


@pytest.mark.parametrize("name", ["dam_a", "dam_b", "dam_c"])
def test_all_cuts_equal_plain(dam_dirs, name):
    reqs = rc.make_requests(td.ALL[name]["vocab"], LENGTHS[name], seed=7)
    want = _oracle(dam_dirs[name], reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    cuts = {"whole": rc.whole(reqs), "tail": rc.bulk_then_tail(reqs, 12), "portions": rc.portions(reqs),
            "mixed": rc.mixed(reqs, seed=3)}
    for cut, steps in cuts.items():
        got = _replay(dam_dirs[name], name, steps)
        worst = max(float(np.abs(got[(rid, p)] - want[rid][p]).max()) for rid, toks in reqs for p in range(len(toks)))
        assert worst <= 5e-5 * scale, f"{name} {cut}: max |dlogit| {worst:.3e} (scale {scale:.3f})"


def test_mixed_reuses_pages_and_state_slots(dam_dirs):
    name = "dam_b"
    reqs = rc.make_requests(td.ALL[name]["vocab"], [40, 33, 70, 21, 64, 18, 50], seed=11)
    steps = rc.mixed(reqs, max_live=3, seed=5)
    assert rc.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for _, t in reqs)
    got = _replay(dam_dirs[name], name, steps, slots=3)  # seven requests through three slots
    want = _oracle(dam_dirs[name], reqs)
    for rid, toks in reqs:
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[rid][p]).max() < 1e-3


def test_config_round_trip_and_layer_runs(tmp_path):
    for name, cfg in td.ALL.items():
        typed = DamolornConfig.from_dict(cfg)
        again = DamolornConfig.from_dict(json.loads(json.dumps(typed.to_dict())))
        assert again == typed
        runs = typed.layer_runs()
        assert runs == plain.layer_order(cfg)
    a = td.typed(td.DAM_A)
    assert [i for i, _ in a.layer_runs()] == [0, 1, 0, 1, 0, 1, 2]
    assert [t for _, t in a.layer_runs()] == [0, None, 1, None, 2, None, None]
    typed = td.typed(td.DAM_C)
    typed.save(tmp_path)
    assert load_config(tmp_path) == typed


def test_config_refusals():
    bad = json.loads(json.dumps(td.DAM_A))
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ConfigError):
        DamolornConfig.from_dict(bad)
    bad = json.loads(json.dumps(td.DAM_A))
    bad["norm"]["groups"] = 5
    with pytest.raises(ConfigError):
        DamolornConfig.from_dict(bad)
    bad = json.loads(json.dumps(td.DAM_A))
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError):
        DamolornConfig.from_dict(bad)
    bad = json.loads(json.dumps(td.DAM_B))
    bad["layers"][0]["mlp"]["router"]["top"] = 7
    with pytest.raises(ConfigError):
        DamolornConfig.from_dict(bad)


def test_parameter_table_names_every_checkpoint_tensor():
    for cfg in td.ALL.values():
        dec = build_decoder(td.typed(cfg))
        named = {src.name: tuple(td.tensor_shapes(cfg)[src.name]) for spec in dec.param_table().values()
                 for src in spec.sources}
        assert named == {k: tuple(v) for k, v in td.tensor_shapes(cfg).items()}


def test_every_layer_run_has_cache_entries_of_its_own():
    dec = build_decoder(td.typed(td.DAM_A))
    entries = dec.cache_entries()
    runs = len(td.typed(td.DAM_A).layer_runs())
    assert len(entries) == 2 * runs  # latent pages and convolution state per run
    ids = [c for call in dec.spec.order for c in call.cache]
    assert sorted(ids) == list(range(2 * runs))
    dec = build_decoder(td.typed(td.DAM_C))  # one tap: nothing but the pages to keep
    assert all(isinstance(call.cache, int) for call in dec.spec.order)


def test_random_weights_folder_loads_and_steps(tmp_path):
    """The random-weights mode writes every tensor the design names (norm gains as ones), and the
    folder loads through the registry and runs a step."""
    from emberserve_b200.engine.runner import StepRow
    from emberserve_b200.weights.loader import write_random_model

    cfg = td.typed(td.DAM_C)
    out = write_random_model(cfg, tmp_path / "m", seed=3, std=0.2)
    _, w = plain.read_model_dir(out)
    assert set(w) == set(td.tensor_shapes(td.DAM_C))
    assert bool((w["l0.norm1"] == 1).all()) and bool((w["final.norm"] == 1).all())
    runner = host_runner(out, page_size=8, num_pages=8, num_state_slots=2)
    runner.cache.admit(0, 5)
    logits = runner.step([StepRow(0, [1, 2, 3, 4, 5], 0, [4])])
    want = plain.forward(td.DAM_C, w, [1, 2, 3, 4, 5], torch.float64)[-1]
    assert (logits[0].double() - want).abs().max() < 1e-4 * want.abs().max()
