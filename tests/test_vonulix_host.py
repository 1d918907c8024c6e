"""Vonulix through the package's own configuration, loader, cache manager, step function and
replay driver on the CPU (the kernels replaced by their restatements), against the plain
implementation: every way of cutting the same requests gives the plain logits."""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import kernel_refs
import plain_vonulix as plain
import replay_cases as rc
import tiny_vonulix as tv
from host_harness import host_runner

from emberserve_b200.config.model import ConfigError
from emberserve_b200.config.vonulix import VonulixConfig
from emberserve_b200.engine.replay import TraceReplayer
from emberserve_b200.parts.base import PagedKV
from emberserve_b200.registry import build_decoder, load_config

LENGTHS = {"von_a": [1, 2, 9, 23, 40, 31], "von_b": [3, 17, 50, 8, 70, 33], "von_c": [2, 48, 11, 61, 35, 5]}


@pytest.fixture(autouse=True)
def _refs(monkeypatch):
    kernel_refs.install(monkeypatch)


@pytest.fixture(scope="module")
def von_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("vonulix")
    return {name: tv.write_model(cfg, root / name, tv.SEEDS[name]) for name, cfg in tv.ALL.items()}


def _replay(model_dir, name, steps, slots=4):
    ps = tv.PAGE_SIZES[name]
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
    assert st.num_sequences == 0 and st.num_free == st.num_pages
    return rc.collect(steps, outs)


def _oracle(model_dir, reqs):
    cfg, w = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, w, toks, torch.float64).numpy() for rid, toks in reqs}


@pytest.mark.parametrize("name", ["von_a", "von_b", "von_c"])
def test_all_cuts_equal_plain(von_dirs, name):
    reqs = rc.make_requests(tv.ALL[name]["vocab"], LENGTHS[name], seed=7)
    want = _oracle(von_dirs[name], reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    cuts = {"whole": rc.whole(reqs), "tail": rc.bulk_then_tail(reqs, 12), "portions": rc.portions(reqs),
            "mixed": rc.mixed(reqs, seed=3)}
    for cut, steps in cuts.items():
        got = _replay(von_dirs[name], name, steps)
        worst = max(float(np.abs(got[(rid, p)] - want[rid][p]).max()) for rid, toks in reqs for p in range(len(toks)))
        assert worst <= 5e-5 * scale, f"{name} {cut}: max |dlogit| {worst:.3e} (scale {scale:.3f})"


def test_mixed_reuses_pages(von_dirs):
    name = "von_b"
    reqs = rc.make_requests(tv.ALL[name]["vocab"], [40, 33, 70, 21, 64, 18, 50], seed=11)
    steps = rc.mixed(reqs, max_live=3, seed=5)
    assert rc.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for _, t in reqs)
    got = _replay(von_dirs[name], name, steps, slots=3)
    want = _oracle(von_dirs[name], reqs)
    for rid, toks in reqs:
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[rid][p]).max() < 1e-3


def test_pages_behind_the_window_go_back_but_not_those_of_the_kept_keys(von_dirs):
    """A window of 7 keys with 3 kept first keys over pages of 4: after 23 tokens the group holds
    the page of positions 0..3 (the kept keys) and the pages from position 16 on (17 is the oldest key
    that the next query reads); the layer with a window of 5 and nothing kept holds pages 4 and 5 only."""
    from emberserve_b200.engine.runner import StepRow

    runner = host_runner(von_dirs["von_a"], page_size=4, num_pages=16, num_state_slots=2)
    toks = list(range(1, 24))
    runner.cache.admit(0, len(toks))
    runner.step([StepRow(0, toks, 0, [len(toks) - 1])])
    groups = {(runner.cache.windows[k], runner.cache.kept_pages[k]): k for k in range(len(runner.cache.windows))}
    held = [p >= 0 for p in runner.cache.table(0, groups[(7, 1)])]
    assert held == [True, False, False, False, True, True]
    held = [p >= 0 for p in runner.cache.table(0, groups[(5, 0)])]
    assert held == [False, False, False, False, True, True]
    runner.cache.check()
    runner.cache.extend(0, 26)
    out = runner.step([StepRow(0, [5, 6, 7], 23, [0, 1, 2])])
    cfg, w = plain.read_model_dir(von_dirs["von_a"])
    want = plain.forward(cfg, w, toks + [5, 6, 7], torch.float64)[-3:]
    assert (out.double() - want).abs().max() < 1e-4 * want.abs().max()
    runner.cache.release(0)
    runner.cache.check()


def test_config_round_trip(tmp_path):
    for cfg in tv.ALL.values():
        typed = VonulixConfig.from_dict(cfg)
        assert VonulixConfig.from_dict(json.loads(json.dumps(typed.to_dict()))) == typed
    typed = tv.typed(tv.VON_B)
    typed.save(tmp_path)
    assert load_config(tmp_path) == typed
    assert typed.layers[0].mixer.rot_factor == 1.0 and typed.layers[1].mixer.rot_factor == 8.0
    assert typed.layers[1].mixer.window is None and typed.layers[3].mlp is None and typed.side_dim == 0
    assert tv.typed(tv.VON_C).layers[0].mlp.shared.limit == 2.0 and tv.typed(tv.VON_C).layers[1].mlp.shared is None


def test_config_refusals():
    def broken(change):
        bad = json.loads(json.dumps(tv.VON_A))
        change(bad)
        with pytest.raises(ConfigError):
            VonulixConfig.from_dict(bad)

    broken(lambda c: c["layers"][0].update(type="something_else"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=4))  # 6 heads over 4
    broken(lambda c: c["layers"][0]["mixer"].update(vdim=7))  # the values turn in pairs
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10))  # more than a head has
    broken(lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0))
    broken(lambda c: c["layers"][0]["mixer"].pop("scale"))
    broken(lambda c: c["layers"][0]["mixer"]["mask"].update(size=0))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=6))  # of 5 experts
    broken(lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"))
    broken(lambda c: c.pop("norm"))


def test_parameter_table_names_every_checkpoint_tensor():
    for cfg in tv.ALL.values():
        dec = build_decoder(tv.typed(cfg))
        named = {src.name: None for spec in dec.param_table().values() for src in spec.sources}
        assert set(named) == set(tv.tensor_shapes(cfg))


def test_cache_entries_per_layer():
    dec = build_decoder(tv.typed(tv.VON_B))
    assert dec.cache_entries() == [PagedKV(4, 16, 40, None, 0, 8), PagedKV(1, 24, None, None, 0, 32),
                                   PagedKV(4, 16, 40, None, 11, 8), PagedKV(2, 8, 16, None, 16, None)]
    assert [call.cache for call in dec.spec.order] == [0, 1, 2, 3]


def test_random_weights_folder_loads_and_steps(tmp_path):
    """The random-weights mode writes every tensor the design names, and the folder loads through
    the registry and runs a step; the rows that pad the gate in the fused projection are zero."""
    from emberserve_b200.engine.runner import StepRow
    from emberserve_b200.weights.loader import write_random_model

    cfg = tv.typed(tv.VON_A)
    out = write_random_model(cfg, tmp_path / "m", seed=3, std=0.2)
    _, w = plain.read_model_dir(out)
    assert set(w) == set(tv.tensor_shapes(tv.VON_A))
    runner = host_runner(out, page_size=8, num_pages=8, num_state_slots=2)
    attn = runner.decoder.blocks[0].mixer
    assert bool((attn.wqkv[attn.gate_at + 6:] == 0).all())
    runner.cache.admit(0, 7)
    logits = runner.step([StepRow(0, [1, 2, 3, 4, 5, 6, 7], 0, [6])])
    want = plain.forward(tv.VON_A, w, [1, 2, 3, 4, 5, 6, 7], torch.float64)[-1]
    assert (logits[0].double() - want).abs().max() < 1e-4 * want.abs().max()
