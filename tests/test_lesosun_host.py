"""Lesosun through the package's own configuration, loader, cache manager, step function and
replay driver on the CPU (the kernels replaced by their restatements), against the plain
implementation: every way of cutting the same requests gives the plain logits."""

from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import kernel_refs
import plain_lesosun as plain
import replay_cases as rc
import tiny_lesosun as tl
from host_harness import host_runner

from emberserve_b200.config.lesosun import ChannelDeltaConfig, LesosunConfig
from emberserve_b200.config.model import ConfigError
from emberserve_b200.engine.replay import TraceReplayer
from emberserve_b200.parts.base import FixedState, PagedKV
from emberserve_b200.registry import build_decoder, load_config

LENGTHS = {"les_a": [1, 2, 9, 23, 40, 31], "les_b": [3, 17, 50, 8, 70, 33], "les_c": [2, 48, 11, 61, 35, 5]}


@pytest.fixture(autouse=True)
def _refs(monkeypatch):
    kernel_refs.install(monkeypatch)


@pytest.fixture(scope="module")
def les_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("lesosun")
    return {name: tl.write_model(cfg, root / name, tl.SEEDS[name]) for name, cfg in tl.ALL.items()}


def _replay(model_dir, name, steps, slots=4):
    ps = tl.PAGE_SIZES[name]
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


@pytest.mark.parametrize("name", ["les_a", "les_b", "les_c"])
def test_all_cuts_equal_plain(les_dirs, name):
    reqs = rc.make_requests(tl.ALL[name]["vocab"], LENGTHS[name], seed=7)
    want = _oracle(les_dirs[name], reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    cuts = {"whole": rc.whole(reqs), "tail": rc.bulk_then_tail(reqs, 12), "portions": rc.portions(reqs),
            "mixed": rc.mixed(reqs, seed=3)}
    for cut, steps in cuts.items():
        got = _replay(les_dirs[name], name, steps)
        worst = max(float(np.abs(got[(rid, p)] - want[rid][p]).max()) for rid, toks in reqs for p in range(len(toks)))
        assert worst <= 5e-5 * scale, f"{name} {cut}: max |dlogit| {worst:.3e} (scale {scale:.3f})"


def test_mixed_reuses_pages_and_state_slots(les_dirs):
    name = "les_b"
    reqs = rc.make_requests(tl.ALL[name]["vocab"], [40, 33, 70, 21, 64, 18, 50], seed=11)
    steps = rc.mixed(reqs, max_live=3, seed=5)
    assert rc.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for _, t in reqs)
    got = _replay(les_dirs[name], name, steps, slots=3)  # seven requests through three slots
    want = _oracle(les_dirs[name], reqs)
    for rid, toks in reqs:
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[rid][p]).max() < 1e-3


def test_portions_of_two_tokens_and_a_long_tail(les_dirs):
    """Portions of two tokens all the way (shorter than every convolution), then forty tokens one by one."""
    name = "les_c"
    reqs = rc.make_requests(tl.ALL[name]["vocab"], [90], seed=21)
    rid, toks = reqs[0]
    steps, at = [], 0
    while at < 50:
        steps.append({"entries": [{"id": rid, "tokens": toks[at:at + 2], "want": [0, 1]}], "end": []})
        at += 2
    while at < len(toks):
        steps.append({"entries": [{"id": rid, "tokens": toks[at:at + 1], "want": [0]}],
                      "end": [rid] if at + 1 == len(toks) else []})
        at += 1
    for n, s in enumerate(steps):
        s["step"] = n
    got = _replay(les_dirs[name], name, steps)
    want = _oracle(les_dirs[name], reqs)[rid]
    scale = float(np.abs(want).max())
    assert max(float(np.abs(got[(rid, p)] - want[p]).max()) for p in range(len(toks))) <= 5e-5 * scale


def test_config_round_trip(tmp_path):
    for cfg in tl.ALL.values():
        typed = LesosunConfig.from_dict(cfg)
        assert LesosunConfig.from_dict(json.loads(json.dumps(typed.to_dict()))) == typed
    typed = tl.typed(tl.LES_B)
    typed.save(tmp_path)
    assert load_config(tmp_path) == typed
    assert typed.logit_softcap is None and tl.typed(tl.LES_A).logit_softcap == 12.0
    assert typed.layers[3].mixer.left.rot_dims == 0 and typed.layers[0].mixer.left.softcap == 3.0
    assert tl.typed(tl.LES_A).layers[2].mixer.left.softcap is None
    assert typed.layers[3].mlp.identity == 3 and typed.layers[1].mlp.shared_ff is None


def test_inner_sizes_come_from_the_checkpoint(les_dirs, tmp_path):
    """A file that does not give the inner sizes of the two-step projections: the tensors' shapes do."""
    cfg = json.loads(json.dumps(tl.LES_A))
    for key in ("decay_rank", "gate_rank"):
        cfg["layers"][0]["mixer"].pop(key)
    bare = LesosunConfig.from_dict(cfg)
    assert bare.layers[0].mixer.decay_rank is None
    with pytest.raises(ConfigError):
        build_decoder(bare)
    _, w = plain.read_model_dir(les_dirs["les_a"])
    out = tl.write_model(cfg, tmp_path / "bare", 0, weights={k: v.to(torch.bfloat16) for k, v in w.items()})
    loaded = load_config(out)
    assert isinstance(loaded.layers[0].mixer, ChannelDeltaConfig)
    assert (loaded.layers[0].mixer.decay_rank, loaded.layers[0].mixer.gate_rank) == (5, 7)
    assert loaded == tl.typed(tl.LES_A)
    cfg["layers"][0]["mixer"]["decay_rank"] = 6  # the file contradicts the tensor
    tl.write_model(cfg, tmp_path / "bare", 0, weights={k: v.to(torch.bfloat16) for k, v in w.items()})
    with pytest.raises(ConfigError):
        load_config(tmp_path / "bare")


def test_config_refusals():
    def broken(change):
        bad = json.loads(json.dumps(tl.LES_A))
        change(bad)
        with pytest.raises(ConfigError):
            LesosunConfig.from_dict(bad)

    broken(lambda c: c["layers"][0].update(type="something_else"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))  # 4 heads over 3
    broken(lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4))  # 6 heads over 4
    broken(lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=10))
    broken(lambda c: c["layers"][1]["mixer"]["left"].pop("scale"))
    broken(lambda c: c["layers"][1]["mixer"]["right"].update(groups=3))  # 4 heads in 3 groups
    broken(lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=5))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=8))  # of 5 + 2
    broken(lambda c: c["layers"][1]["mlp"].update(kind="sparse"))
    broken(lambda c: c.pop("norm"))
    broken(lambda c: c.update(logit_softcap=-1.0))


def test_parameter_table_names_every_checkpoint_tensor():
    for cfg in tl.ALL.values():
        dec = build_decoder(tl.typed(cfg))
        named = {src.name: None for spec in dec.param_table().values() for src in spec.sources}
        assert set(named) == set(tl.tensor_shapes(cfg))


def test_cache_entries_per_layer():
    dec = build_decoder(tl.typed(tl.LES_A))
    entries = dec.cache_entries()
    # delta: convolution inputs + memory; parallel: pages, attention's convolution, state space's convolution,
    # its state; parallel whose convolutions have one tap: pages and state alone
    assert [type(e) for e in entries] == [FixedState, FixedState, PagedKV, FixedState, FixedState, FixedState,
                                          PagedKV, FixedState]
    assert [call.cache for call in dec.spec.order] == [(0, 1), (2, 3, 4, 5), (6, 7)]
    assert entries[0] == FixedState((2, 2 * 16 + 48), "float32") and entries[1] == FixedState((4, 8 * 12), "float32")
    assert entries[2] == PagedKV(2, 8, None, None, v_head_dim=16) and entries[6] == PagedKV(2, 16, None, None)
    assert entries[3] == FixedState((1, 6 * 8 + 2 * 8 + 2 * 16), "float32")
    assert entries[4] == FixedState((3, 24 + 2 * 10), "float32") and entries[5] == FixedState((4, 5 * 6), "float32")


def test_random_weights_folder_loads_and_steps(tmp_path):
    """The random-weights mode writes every tensor the design names, and the folder loads through
    the registry and runs a step; the rows that pad the fused projections are zero."""
    from emberserve_b200.engine.runner import StepRow
    from emberserve_b200.weights.loader import write_random_model

    cfg = tl.typed(tl.LES_A)
    out = write_random_model(cfg, tmp_path / "m", seed=3, std=0.2)
    _, w = plain.read_model_dir(out)
    assert set(w) == set(tl.tensor_shapes(tl.LES_A))
    runner = host_runner(out, page_size=8, num_pages=8, num_state_slots=2)
    delta = runner.decoder.blocks[0].mixer
    assert bool((delta.win[delta.a_at + 5:delta.g_at] == 0).all()) and bool((delta.win[delta.b_at + 4:] == 0).all())
    ssm = runner.decoder.blocks[1].mixer.right
    assert bool((ssm.win[ssm.rows:] == 0).all())
    runner.cache.admit(0, 7)
    logits = runner.step([StepRow(0, [1, 2, 3, 4, 5, 6, 7], 0, [6])])
    want = plain.forward(tl.LES_A, w, [1, 2, 3, 4, 5, 6, 7], torch.float64)[-1]
    assert (logits[0].double() - want).abs().max() < 1e-4 * want.abs().max()


def test_identity_experts_and_correction_change_the_choice(les_dirs):
    """The plain router: a correction large enough moves the choice while the weights stay the scores; an
    identity expert returns its input."""
    cfg, w = plain.read_model_dir(les_dirs["les_b"])
    w = {k: v.double() for k, v in w.items()}
    mlp, p = cfg["layers"][3]["mlp"], "l3.mlp."
    gen = torch.Generator().manual_seed(5)
    h = torch.randn(6, cfg["width"], generator=gen, dtype=torch.float64)
    seen = []
    base = plain.routed_ff(h, w, p, mlp, seen)
    w2 = dict(w)
    w2[p + "correction"] = w[p + "correction"].clone()
    w2[p + "correction"][-1] += 10.0  # the last identity expert is now always chosen
    seen2 = []
    moved = plain.routed_ff(h, w2, p, mlp, seen2)
    assert bool((seen2[0][1] == mlp["router"]["experts"] + mlp["router"]["identity"] - 1).any(-1).all())
    assert not torch.allclose(base, moved)
