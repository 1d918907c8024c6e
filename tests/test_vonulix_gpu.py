"""Vonulix on the GPU: every mechanism's kernels alone against their restatements and against the plain
implementation (``plain_vonulix``); keys that one score singles out just inside and just outside the
window, among the kept first keys and just behind them, at page borders, far back and first in a
sequence, in prompts and in decoding; the engine under every way of cutting the same requests, batches
against each request alone, pools whose pages change hands, long decoding, the sizes that the
tensor-core kernels take, and greedy generation through the entry point and its scheduler."""

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
import plain_vonulix as plain
import replay_cases as rc
import tiny_vonulix as tv

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
LENGTHS = {"von_a": [1, 2, 9, 23, 40, 31, 130], "von_b": [3, 17, 50, 8, 70, 33, 150],
           "von_c": [2, 48, 11, 61, 35, 5, 97]}
TOL32 = 5e-5  # of the largest |logit|
TOL16 = 6e-2  # bfloat16 against the 64-bit plain implementation, weights drawn wide
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _K():
    from emberserve_b200 import kernels

    return kernels


def _close(got, want, dtype, what="", tol16=1.2e-2):
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    scale = float(want.abs().max()) + 1e-30
    tol = 2e-5 if dtype == torch.float32 else tol16
    err = float((got - want).abs().max()) / scale
    assert err <= tol, f"{what}: {err:.3e} of scale {scale:.3e}"


def _turn_table(n, base, positions, factor=1.0):
    """[positions, n / 2, (cos, sin)] of the angles pos * base^(-2i/n) / factor, as the package lays it out."""
    ang = torch.arange(positions, dtype=torch.float64)[:, None] * plain.pair_frequencies(n, base, torch.float64)[None, :] / factor
    return torch.stack((torch.cos(ang), torch.sin(ang)), -1).float()


@pytest.fixture(scope="module")
def von_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("vonulix")
    return {name: tv.write_model(cfg, root / name, tv.SEEDS[name]) for name, cfg in tv.ALL.items()}


# ---- kernels alone ----------------------------------------------------------------------------

def _paged(g, dtype, nkv, d, dv, page_size, ctx_lens):
    """Block tables over shuffled pages for requests of the given lengths; stale contents everywhere."""
    pages_per = [-(-c // page_size) for c in ctx_lens]
    total = sum(pages_per) + 3
    perm = torch.randperm(total, generator=g).tolist()
    bt = torch.zeros(len(ctx_lens), max(pages_per), dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    kc = torch.randn(total, nkv, page_size, d, generator=g).to(dtype)
    vc = torch.randn(total, nkv, page_size, dv, generator=g).to(dtype)
    return bt, kc, vc


@DTYPES
@pytest.mark.parametrize("rot,d,dv", [(4, 8, 16), (16, 16, 8), (6, 24, 32), (32, 64, 64), (0, 8, 8)])
def test_unit_values_turned_by_their_position_as_they_are_cached(dtype, rot, d, dv):
    g = torch.Generator().manual_seed(rot + d + dv)
    nh, nkv, ps = 6, 2, 4
    starts, qlens = [0, 9, 3], [7, 1, 5]
    bt, kc, vc = _paged(g, dtype, nkv, d, dv, ps, [s + q for s, q in zip(starts, qlens)])
    n = sum(qlens)
    proj = torch.randn(n, (nh + nkv) * d + nkv * dv + 8, generator=g).to(dtype)
    posl = np.concatenate([np.arange(s, s + q) for s, q in zip(starts, qlens)])
    pos, row_of = _i32(posl), _i32(np.repeat(np.arange(3), qlens))
    table = _turn_table(rot, 50.0, 32, 2.5) if rot else None
    vtable = _turn_table(dv, 50.0, 32)
    want = (proj.clone(), kc.clone(), vc.clone())
    R.qk_prep(want[0], nh, nkv, d, pos.cpu(), row_of.cpu(), table, rot, "half", None, want[1], want[2], bt, False,
              v_norm_eps=1e-5, v_table=vtable)
    got = (proj.to(DEV), kc.to(DEV), vc.to(DEV))
    _K().qk_prep(got[0], nh, nkv, d, pos, row_of, None if table is None else table.to(DEV), rot, "half", None,
                 got[1], got[2], bt.to(DEV), False, v_norm_eps=1e-5, v_table=vtable.to(DEV))
    for a, b, what in zip(got, want, ("q", "k cache", "v cache")):
        _close(a, b, dtype, what)
    # against the plain mechanisms: a token of request 2 at position 3 + 4
    t, p = 8 + 4, 7
    page, slot = int(bt[2, p // ps]), p % ps
    ang = torch.full((1, dv // 2), float(p), dtype=torch.float64) * plain.pair_frequencies(dv, 50.0, torch.float64)
    v = proj[t, (nh + nkv) * d:(nh + nkv) * d + nkv * dv].double().view(1, nkv, dv)
    _close(got[2][page, :, slot], plain.turn_halves(plain.unit_rms(v, 1e-5), ang)[0], dtype, "value against plain")
    if rot:
        ang = torch.full((1, rot // 2), float(p), dtype=torch.float64) * plain.pair_frequencies(rot, 50.0, torch.float64) / 2.5
        k = proj[t, nh * d:(nh + nkv) * d].double().view(1, nkv, d)
        _close(got[1][page, :, slot], plain.turn_halves(k, ang)[0], dtype, "key against plain")


def _attention_case(g, dtype, nh, nkv, d, dv, ps, starts, qlens):
    ctx = [s + q for s, q in zip(starts, qlens)]
    bt, kc, vc = _paged(g, dtype, nkv, d, dv, ps, ctx)
    n = sum(qlens)
    q = torch.randn(n, nh * d + 16, generator=g).to(dtype)
    gate = torch.randn(n, nh + 3, generator=g).to(dtype)
    cu = _i32(np.concatenate([[0], np.cumsum(qlens)]))
    pos = _i32(np.concatenate([np.arange(s, s + q) for s, q in zip(starts, qlens)]))
    return q, gate, pos, bt, kc, vc, cu, _i32(starts), n


def _run_attention(case, nh, nkv, d, scale, max_q, rows, window, keep, table, use_gate=True, splits=1, dev=True,
                   kernel="auto"):
    q, gate, pos, bt, kc, vc, cu, st, n = case
    dv = vc.shape[3]
    mod = _K() if dev else R
    mv = (lambda t: t.to(DEV)) if dev else (lambda t: t.cpu())
    out = torch.zeros(n, nh * dv, dtype=q.dtype, device=DEV if dev else "cpu")
    scratch = None
    if splits > 1 and dev:
        scratch = torch.empty(mod.attention_scratch_bytes(n, nh, dv, splits) // 4, dtype=torch.float32, device=DEV)
    mod.paged_attention_masked(mv(q), out, mv(kc), mv(vc), mv(bt), mv(cu), mv(st), rows, n, nh, nkv, d, scale, max_q,
                               window=window, gate=mv(gate) if use_gate else None, splits=splits, scratch=scratch,
                               keep_first=keep, out_table=None if table is None else mv(table), positions=mv(pos),
                               kernel=kernel)
    return out


ATTENTION_SIZES = [(6, 2, 8, 16, 4, 7, 3), (4, 4, 16, 8, 16, 40, 11), (5, 1, 24, 24, 8, 1, 9), (2, 1, 24, 32, 16, None, 0),
                   (8, 2, 8, 8, 16, 16, 16), (9, 3, 64, 64, 16, 40, 5), (3, 3, 128, 128, 32, 100, 70),
                   (8, 1, 64, 64, 8, 33, 64), (4, 2, 64, 64, 16, 64, 1), (2, 2, 64, 32, 16, 20, 4),
                   (32, 1, 64, 64, 16, 50, 6), (2, 2, 96, 32, 16, 30, 2), (1, 1, 256, 256, 16, 130, 3)]


@DTYPES
@pytest.mark.parametrize("nh,nkv,d,dv,ps,window,keep", ATTENTION_SIZES)
def test_window_with_kept_first_keys_and_turned_values_against_dense(dtype, nh, nkv, d, dv, ps, window, keep):
    g = torch.Generator().manual_seed(nh * d + dv)
    table = _turn_table(dv, 300.0, 400)
    starts, qlens = [0, 61, 17, 230, 5, 0], [33, 1, 20, 1, 2, 150]  # prompts, portions and single tokens in one step
    case = _attention_case(g, dtype, nh, nkv, d, dv, ps, starts, qlens)
    for tab, use_gate in ((table, True), (None, True), (table, False)):
        want = _run_attention(case, nh, nkv, d, 0.4, max(qlens), 6, window, keep, tab, use_gate, dev=False)
        got = _run_attention(case, nh, nkv, d, 0.4, max(qlens), 6, window, keep, tab, use_gate)
        _close(got, want, dtype, f"turned={tab is not None} gate={use_gate}")
    # single tokens only, keys split over blocks and merged
    starts, qlens = [300, 7, 64, 0, 129], [1, 1, 1, 1, 1]
    case = _attention_case(g, dtype, nh, nkv, d, dv, ps, starts, qlens)
    want = _run_attention(case, nh, nkv, d, 0.4, 1, 5, window, keep, table, dev=False)
    for splits in (1, 2, 5):
        got = _run_attention(case, nh, nkv, d, 0.4, 1, 5, window, keep, table, splits=splits)
        _close(got, want, dtype, f"splits={splits}")


@DTYPES
@pytest.mark.parametrize("d", [16, 64, 128], ids=["generic", "tensor-core-64", "tensor-core-128"])
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
def test_a_planted_key_shows_at_the_edges_of_the_window_and_of_the_kept_keys(dtype, decode, d):
    """One key is made to win the softmax (its dot product with one query stands out) and its value is
    large: the size of the output shows whether the query saw it.  A window of 40 keys (no multiple of
    the page of 16) that keeps the first 5: from position 200 the keys 161..200 are seen, 160 is not;
    keys 0..4 are seen, 5 is not; nor is a key far back between them; the first key of a page is, and
    the query itself.  The values stay as cached (no turning), so that the one-hot shows directly."""
    nh, nkv, ps, window, keep = 2, 1, 16, 40, 5
    g = torch.Generator().manual_seed(5)
    qpos = 200
    for key, seen in ((161, True), (160, False), (4, True), (5, False), (0, True), (100, False), (176, True),
                      (200, True), (159, False), (15, False), (16, False)):
        start, qlen = (qpos, 1) if decode else (qpos - 9, 12)
        case = list(_attention_case(g, dtype, nh, nkv, d, d, ps, [start], [qlen]))
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
        out = _run_attention(case, nh, nkv, d, 4.0 / d, qlen, 1, window, keep, None, use_gate=False)
        got = float(out[row, 3])
        assert (got > 40.0) == seen, f"key {key} from position {qpos}: {got}"
        want = _run_attention(case, nh, nkv, d, 4.0 / d, qlen, 1, window, keep, None, use_gate=False, dev=False)
        _close(out, want, dtype, f"key {key}")
        if decode:  # the same with the keys split over blocks
            out = _run_attention(case, nh, nkv, d, 4.0 / d, 1, 1, window, keep, None, use_gate=False, splits=3)
            assert (float(out[row, 3]) > 40.0) == seen, f"key {key}, split"


@DTYPES
@pytest.mark.parametrize("d", [8, 64])
def test_a_far_key_among_hundreds_and_the_first_tokens(dtype, d):
    """Without a window a key 700 positions back is seen (planted as above); with the kept keys reaching past
    the whole context (keep >= context) nothing is hidden either; and the first token of a sequence sees
    itself alone: its output is its own value, turned by zero."""
    nh, nkv, ps = 2, 2, 16
    g = torch.Generator().manual_seed(8)
    table = _turn_table(d, 100.0, 800)
    for window, keep in ((None, 0), (3, 750)):
        case = list(_attention_case(g, dtype, nh, nkv, d, d, ps, [741], [1]))
        q, bt, kc, vc = case[0], case[3], case[4].float() * 0.1, case[5].float() * 0.1
        q[0, :nh * d] = 0
        q[0, :d] = 4.0
        page, slot = int(bt[0, 41 // ps]), 41 % ps
        kc[page, 0, slot] = 4.0
        vc[page, 0, slot] = 0
        vc[page, 0, slot, 2] = 50.0
        case[4], case[5] = kc.to(dtype), vc.to(dtype)
        out = _run_attention(case, nh, nkv, d, 4.0 / d, 1, 1, window, keep, None, use_gate=False)
        assert float(out[0, 2]) > 40.0
        out = _run_attention(case, nh, nkv, d, 4.0 / d, 1, 1, window, keep, table, use_gate=False)
        want = _run_attention(case, nh, nkv, d, 4.0 / d, 1, 1, window, keep, table, use_gate=False, dev=False)
        _close(out, want, dtype, "turned back over 700 positions")
        assert float(out[0, :d].float().norm()) > 40.0
    case = _attention_case(g, dtype, nh, nkv, d, d, ps, [0], [1])
    out = _run_attention(case, nh, nkv, d, 0.3, 1, 1, 5, 2, table, use_gate=False)
    page = int(case[3][0, 0])
    _close(out.view(nh, d), case[5][page, :, 0], dtype, "the first token")


def _route_and_run(x, router, wgu, wdown, top, limit, dtype):
    """The kernels of routed experts in the order the part calls them (scores multiply the inputs)."""
    K = _K()
    n, e = x.shape[0], router.shape[0]
    ff, hid = wgu.shape[1] // 2, x.shape[1]
    pairs = n * top
    logits = x.float() @ router.float().t()
    tiles = K.moe_max_tiles(pairs, e, K.moe_tile_rows())
    ids, perm = (torch.zeros(pairs, dtype=torch.int32, device=DEV) for _ in range(2))
    weights = torch.zeros(pairs, device=DEV)
    offsets = torch.zeros(3 * e + 1, dtype=torch.int32, device=DEV)
    plan = torch.zeros(1 + 3 * tiles, dtype=torch.int32, device=DEV)
    K.moe_route(logits, top, False, ids, weights, offsets, perm, plan, tiles, scoring="sigmoid")
    act = torch.zeros(pairs, ff, dtype=dtype, device=DEV)
    K.moe_up(x, wgu, perm, offsets, plan, tiles, top, "swiglu_capped", act, in_scale=weights, limit=limit, alpha=1.702)
    y = torch.zeros(pairs, hid, device=DEV)
    K.moe_down(act, wdown, perm, offsets, plan, tiles, y)
    out = torch.zeros(n, hid, dtype=dtype, device=DEV)
    K.moe_combine(y, None, out, top)
    return out, ids.view(n, top), weights.view(n, top)


@DTYPES
@pytest.mark.parametrize("n,e,top,hid,ff,limit", [(37, 5, 2, 48, 24, 1.5), (1, 12, 1, 64, 80, 2.2), (200, 9, 1, 40, 8, 0.7),
                                                  (70, 6, 4, 40, 12, 4.0), (130, 3, 3, 64, 32, 2.5), (600, 8, 2, 128, 64, 1.0),
                                                  (50, 1, 1, 32, 16, 1.0), (9, 2, 1, 36, 20, 3.0)])
def test_sigmoid_scored_experts_whose_scores_multiply_their_inputs(dtype, n, e, top, hid, ff, limit):
    g = torch.Generator().manual_seed(n + e)
    x = torch.randn(n, hid, generator=g).to(dtype)
    w = {"router": (torch.randn(e, hid, generator=g) * 0.3).to(dtype)}
    for j in range(e):
        w[f"e{j}.gate"] = (torch.randn(ff, hid, generator=g) * 1.5 / math.sqrt(hid)).to(dtype)
        w[f"e{j}.up"] = (torch.randn(ff, hid, generator=g) * 1.5 / math.sqrt(hid)).to(dtype)
        w[f"e{j}.down"] = (torch.randn(hid, ff, generator=g) / math.sqrt(ff)).to(dtype)
    wgu = torch.stack([torch.cat((w[f"e{j}.gate"], w[f"e{j}.up"])) for j in range(e)]).to(DEV)
    wdown = torch.stack([w[f"e{j}.down"] for j in range(e)]).to(DEV)
    got, ids, weights = _route_and_run(x.to(DEV), w["router"].to(DEV), wgu, wdown, top, limit, dtype)
    m = {"router": {"experts": e, "top": top}, "expert": {"limit": limit}}
    want = plain.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, "", m)
    s = torch.sigmoid(x.double() @ w["router"].double().t())
    order = torch.argsort(-s, dim=-1, stable=True)[:, :top]
    assert torch.equal(ids.cpu().long(), order)
    _close(weights, torch.gather(s, 1, order), torch.float32, "the scores as they are")
    _close(got, want, dtype, "experts", tol16=2.5e-2)


def test_experts_of_a_long_prompt_on_the_grouped_tensor_core_product():
    """More than 512 tokens in bfloat16: the pairs are laid out in groups of 256 rows per expert, gathered,
    and both products run in their grouped tcgen05 form, the scores on the 32-bit sums and the capped
    activation in the first one's epilogue, a shared expert's rows added at the end."""
    K = _K()
    g = torch.Generator().manual_seed(12)
    for n, e, top, hid, ff, limit in ((700, 5, 2, 64, 128, 1.5), (1500, 16, 1, 192, 256, 2.0), (520, 3, 3, 128, 128, 0.6)):
        x = torch.randn(n, hid, generator=g).to(torch.bfloat16)
        w = {"router": (torch.randn(e, hid, generator=g) * 0.3).to(torch.bfloat16)}
        for j in range(e):
            w[f"e{j}.gate"] = (torch.randn(ff, hid, generator=g) * 1.5 / math.sqrt(hid)).to(torch.bfloat16)
            w[f"e{j}.up"] = (torch.randn(ff, hid, generator=g) * 1.5 / math.sqrt(hid)).to(torch.bfloat16)
            w[f"e{j}.down"] = (torch.randn(hid, ff, generator=g) / math.sqrt(ff)).to(torch.bfloat16)
        wgu = torch.stack([torch.cat((w[f"e{j}.gate"], w[f"e{j}.up"])) for j in range(e)]).to(DEV)
        wdown = torch.stack([w[f"e{j}.down"] for j in range(e)]).to(DEV)
        extra = torch.randn(n, hid, generator=g).to(torch.bfloat16)
        xd, pairs = x.to(DEV), n * top
        logits = xd.float() @ w["router"].to(DEV).float().t()
        tiles = K.moe_max_tiles(pairs, e, K.moe_tile_rows())
        big = torch.zeros(K.moe_max_tiles(pairs, e, K.MOE_BIG_TILE_ROWS), dtype=torch.int32, device=DEV)
        rows = big.numel() * K.MOE_BIG_TILE_ROWS
        ids, inv = (torch.zeros(pairs, dtype=torch.int32, device=DEV) for _ in range(2))
        perm = torch.zeros(rows, dtype=torch.int32, device=DEV)
        weights = torch.zeros(pairs, device=DEV)
        offsets = torch.zeros(3 * e + 1, dtype=torch.int32, device=DEV)
        plan = torch.zeros(1 + 3 * tiles, dtype=torch.int32, device=DEV)
        K.moe_route(logits, top, False, ids, weights, offsets, perm, plan, tiles, align=K.MOE_BIG_TILE_ROWS, big=big,
                    inv=inv, scoring="sigmoid")
        xs = torch.zeros(rows, hid, dtype=torch.bfloat16, device=DEV)
        K.moe_gather(xd, perm, top, xs)
        act = torch.zeros(rows, ff, dtype=torch.bfloat16, device=DEV)
        K.moe_up_grouped_tc05(xs, wgu, big, act, "swiglu_capped", perm, weights, limit, 1.702)
        y16 = torch.zeros(rows, hid, dtype=torch.bfloat16, device=DEV)
        K.moe_down_grouped_tc05(act, wdown, big, y16)
        out = torch.zeros(n, hid, dtype=torch.bfloat16, device=DEV)
        K.moe_combine_rows(y16, inv, None, out, top, extra=extra.to(DEV))
        m = {"router": {"experts": e, "top": top}, "expert": {"limit": limit}}
        want = plain.routed_experts(x.double(), {k: v.double() for k, v in w.items()}, "", m) + extra.double()
        _close(out, want, torch.bfloat16, f"{n} tokens, {e} experts", tol16=2.5e-2)


@DTYPES
def test_capped_activation_and_the_gate_per_token(dtype):
    """g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1); with the row's
    own sigmoid number (the shared expert's gate) on top.  Inputs reach well past the limits."""
    g = torch.Generator().manual_seed(3)
    for i, limit in ((24, 0.8), (88, 1.1), (40, 7.0)):
        gu = (3 * torch.randn(19, 2 * i + 8, generator=g)).to(dtype)
        a, b = gu[:, :i].double().clamp(max=limit), gu[:, i:2 * i].double().clamp(-limit, limit)
        want = a * torch.sigmoid(1.702 * a) * (b + 1)
        got = torch.empty(19, i, dtype=dtype, device=DEV)
        _K().glu_act(gu.to(DEV), got, "swiglu_capped", limit, 1.702)
        _close(got, want, dtype, f"limit {limit}")
        _K().glu_act(gu.to(DEV), got, "swiglu_capped", limit, 1.702, row_gate=True)
        _close(got, want * torch.sigmoid(gu[:, 2 * i].double())[:, None], dtype, f"limit {limit}, gated rows")


@DTYPES
def test_token_input_and_depth_average_kernels(dtype):
    """gelu_tanh(z) * (the token's columns of the second table); the stream's newest state joined to the
    history (a normed delta added) and the weighted sum over all depths so far, in 32 bits."""
    g = torch.Generator().manual_seed(4)
    n, c, h, depths = 13, 9, 40, 4
    z = (2 * torch.randn(n, c, generator=g)).to(dtype)
    table = torch.randn(30, 5 * c, generator=g).to(dtype)
    tokens = torch.randint(0, 30, (n,), generator=g)
    got = torch.empty(n, c, dtype=dtype, device=DEV)
    _K().token_gate(z.to(DEV), table.to(DEV), 2 * c, tokens.to(torch.int32).to(DEV), got)
    _close(got, plain.gelu_tanh(z.double()) * table[tokens][:, 2 * c:3 * c].double(), dtype, "token gate")
    for h in (40, 42, 2048):  # four columns per thread where the width allows, one otherwise
        _depth_average_case(g, dtype, n, h, depths)
    # the stream itself as an operand: the add in 32 bits, rounded once
    res = torch.randn(n, h, generator=g)
    delta = torch.randn(n, h, generator=g).to(dtype)
    dr, xb = res.to(DEV), torch.empty(n, h, dtype=dtype, device=DEV)
    _K().add_cast(delta.to(DEV), dr, xb)
    _close(dr, res.double() + delta.double(), torch.float32, "sum")
    assert torch.equal(xb.cpu(), (res + delta.float()).to(dtype))


def _depth_average_case(g, dtype, n, h, depths):
    hist = torch.randn(depths + 1, n, h, generator=g)
    res = torch.randn(n, h, generator=g)
    for count, normed in ((1, False), (2, True), (3, False), (5, True)):
        delta = torch.randn(n, h, generator=g).to(dtype) if count > 1 else None
        gain = torch.randn(h, generator=g).to(dtype) if normed else None
        w = torch.randn(count, generator=g) if count > 1 else None
        x = res.double()
        if delta is not None:
            x = x + (plain.unit_rms(delta.double(), 1e-5) * gain.double() if normed else delta.double())
        states = [hist[j].double() for j in range(count - 1)] + [x]
        want = x if w is None else sum(w[j].double() * states[j] for j in range(count))
        dh, dr = hist.to(DEV), res.to(DEV)
        _K().depth_mix(None if delta is None else delta.to(DEV), None if gain is None else gain.to(DEV), 1e-5, dr, dh,
                       None if w is None else w.to(DEV), count)
        _close(dr, want, torch.float32, f"depth {count}")
        _close(dh[count - 1], x, torch.float32, f"state {count}")
        assert torch.equal(dh[:count - 1].cpu(), hist[:count - 1]) and torch.equal(dh[count:].cpu(), hist[count:])


# ---- the engine -------------------------------------------------------------------------------

def _oracle(model_dir, reqs):
    cfg, w = plain.read_model_dir(model_dir)
    return {rid: plain.forward(cfg, w, toks, torch.float64).numpy() for rid, toks in reqs}


def _replay(model_dir, name, dtype, steps, slots=4, page_size=None, attn_kernel="auto"):
    from emberserve_b200.engine.replay import TraceReplayer
    from emberserve_b200.engine.runner import ModelRunner

    ps = page_size or tv.PAGE_SIZES[name]
    pages = TraceReplayer.pages_for(rc.max_live_tokens(steps), ps)
    runner = ModelRunner.from_dir(model_dir, dtype, page_size=ps, num_pages=pages, num_state_slots=slots)
    runner.attn_kernel = attn_kernel
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


def _compare(got, want, reqs, scale, dtype, what):
    errs = np.array([float(np.abs(got[(rid, p)] - want[rid][p]).max()) for rid, toks in reqs
                     for p in range(len(toks))]) / scale
    if dtype == torch.float32:
        assert errs.max() <= TOL32, f"{what}: max |dlogit| / scale {errs.max():.3e}"
    else:
        # In bfloat16 the router reads a rounded input: where two experts' scores nearly tie, the rounding
        # may choose the other one, and that position's logits move by much more than rounding.  Such
        # positions (and later ones that attend to them) are few; the 32-bit runs are exact at every position.
        over = int((errs > TOL16).sum())
        assert over <= max(1, len(errs) // 20) and np.median(errs) <= TOL16 / 4 and np.quantile(errs, 0.9) <= TOL16 / 2, (
            f"{what}: {over} of {len(errs)} over, max {errs.max():.3e}, median {np.median(errs):.3e}")


# one mechanism per model: a layer that is its attention alone (at a generic and at a tensor-core head size,
# with and without window, kept keys and scaling), one with routed experts alone or beside a shared expert,
# and the token input and the depth average around the smallest layer
ONE_LAYER = {
    "attention": (tv._layer(tv._mixer(4, 2, 16, 8, 9, 2, 8, 1000.0, 2.0), None), None),
    "attention_64": (tv._layer(tv._mixer(4, 2, 64, 64, 20, 5, 16, 5000.0, 2.0), None), None),
    "attention_128": (tv._layer(tv._mixer(2, 1, 128, 128, 70, 17, 128, 5000.0), None), None),
    "attention_unbounded": (tv._layer(tv._mixer(3, 1, 64, 64, None, 0, 16, 100.0), None), None),
    "experts": (tv._layer(tv._mixer(1, 1, 8, 8, None, 0, 0, 10.0), tv._moe(7, 2, 16, 1.2)), None),
    "experts_shared": (tv._layer(tv._mixer(1, 1, 8, 8, None, 0, 0, 10.0), tv._moe(4, 1, 16, 0.9, (24, 2.0))), None),
    "token_input": (tv._layer(tv._mixer(1, 1, 8, 8, 4, 0, 2, 10.0), None), 6),
}


@DTYPES
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_one_layer_models_in_prompt_and_token_by_token(tmp_path, which, dtype):
    layer, side = ONE_LAYER[which]
    cfg = {"architecture": "Vonulix", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "max_positions": 256,
           "embedding": {"scale": 2.0}, "layers": [layer, layer]}
    if side:
        cfg["token_side"] = {"dim": side}
    model = tv.write_model(cfg, tmp_path / which, 31)
    reqs = rc.make_requests(50, [45, 140], seed=1)
    want = _oracle(model, reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    for steps in (rc.whole(reqs), rc.bulk_then_tail(reqs, 100), rc.portions(reqs)):
        got = _replay(model, None, dtype, steps, page_size=16)
        _compare(got, want, reqs, scale, dtype, which)


@pytest.fixture(scope="module")
def cases(von_dirs):
    out = {}
    for name in tv.ALL:
        reqs = rc.make_requests(tv.ALL[name]["vocab"], LENGTHS[name], seed=7)
        want = _oracle(von_dirs[name], reqs)
        out[name] = (reqs, want, max(float(np.abs(v).max()) for v in want.values()))
    return out


@DTYPES
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["von_a", "von_b", "von_c"])
def test_cut_equals_plain(von_dirs, cases, name, cut, dtype):
    reqs, want, scale = cases[name]
    steps = {"whole": rc.whole, "tail": lambda r: rc.bulk_then_tail(r, 40), "portions": rc.portions,
             "mixed": lambda r: rc.mixed(r, seed=3)}[cut](reqs)
    if cut == "mixed":
        assert rc.max_live_tokens(steps) < sum(-(-len(t) // 64) * 64 for _, t in reqs)
    got = _replay(von_dirs[name], name, dtype, steps)
    assert len(got) == sum(len(t) for _, t in reqs)
    _compare(got, want, reqs, scale, dtype, f"{name} {cut}")


def test_batches_of_unequal_requests_equal_each_alone(von_dirs, cases):
    """In 32 bits a request's logits in a mixed batch, through a small pool that seven requests share in
    turn, are those it has alone."""
    name = "von_b"
    reqs, want, scale = cases[name]
    alone = _replay(von_dirs[name], name, torch.float32, rc.whole(reqs))
    mixed = _replay(von_dirs[name], name, torch.float32, rc.mixed(reqs, max_live=3, seed=9), slots=3)
    worst = max(float(np.abs(alone[k] - mixed[k]).max()) for k in alone)
    assert worst <= TOL32 * scale


@DTYPES
def test_long_decoding_token_by_token(von_dirs, dtype):
    """A whole request one token per step, from the first token on (a one-key softmax), across many pages,
    past the kept keys and past windows of 7 and 5 keys."""
    name = "von_a"
    reqs = rc.make_requests(tv.ALL[name]["vocab"], [150], seed=21)
    want = _oracle(von_dirs[name], reqs)
    scale = float(np.abs(want["r0"]).max())
    got = _replay(von_dirs[name], name, dtype, rc.bulk_then_tail(reqs, 150))
    _compare(got, want, reqs, scale, dtype, "token by token")


# head sizes that the tensor-core kernels take, windows that are no multiple of a page or of a key tile,
# kept keys inside a tile and past one, six and one query heads per key head
VON_T = {
    "architecture": "Vonulix", "vocab": 120, "width": 64, "norm": {"eps": 1e-6}, "max_positions": 1024,
    "embedding": {"scale": 4.0}, "token_side": {"dim": 8},
    "layers": [
        tv._layer(tv._mixer(6, 1, 64, 64, 90, 7, 48, 30000.0, 3.0, 0.2), tv._moe(6, 2, 32, 2.0, (32, 1.0))),
        tv._layer(tv._mixer(2, 2, 128, 128, 150, 70, 64, 10000.0), None),
        tv._layer(tv._mixer(4, 2, 64, 64, 33, 0, 64, 100.0, 2.0), tv._moe(5, 1, 48, 1.0)),
    ],
}


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_tensor_core_head_sizes_against_plain_and_against_the_generic_kernel(tmp_path_factory, cut):
    model = tv.write_model(VON_T, tmp_path_factory.mktemp("von_t"), 40)
    reqs = rc.make_requests(VON_T["vocab"], [300, 71, 2, 190, 415], seed=13)
    want = _oracle(model, reqs)
    scale = max(float(np.abs(v).max()) for v in want.values())
    steps = {"whole": rc.whole, "tail": lambda r: rc.bulk_then_tail(r, 170), "mixed": lambda r: rc.mixed(r, seed=6),
             "portions": lambda r: rc.portions(r, (37, 5, 64, 2, 110, 3))}[cut](reqs)
    got32 = _replay(model, None, torch.float32, steps, page_size=16)
    _compare(got32, want, reqs, scale, torch.float32, f"float32 {cut}")
    got = _replay(model, None, torch.bfloat16, steps, page_size=16)
    _compare(got, want, reqs, scale, torch.bfloat16, f"bfloat16 {cut}")
    generic = _replay(model, None, torch.bfloat16, steps, page_size=16, attn_kernel="generic")
    errs = np.array([float(np.abs(got[k] - generic[k]).max()) for k in got]) / scale
    # (two bfloat16 runs may choose another expert where two scores nearly tie, as in `_compare`)
    over = int((errs > TOL16 / 2).sum())
    assert over <= max(1, len(errs) // 50) and np.median(errs) <= TOL16 / 8, f"{cut}: {over} over, {errs.max():.3e} {np.median(errs):.3e}"


def test_a_long_prompt_whole_and_in_portions(tmp_path):
    """A prompt of 900 tokens in one step (the experts on the grouped tensor-core products, attention over
    many key tiles, kept keys far behind the window) against the plain implementation and against the
    same prompt in portions of at most 300 tokens."""
    cfg = json.loads(json.dumps(VON_T))
    cfg["layers"][0]["mlp"] = tv._moe(6, 2, 128, 2.0, (128, 1.0))
    cfg["layers"][2]["mlp"] = tv._moe(5, 1, 256, 1.0)
    model = tv.write_model(cfg, tmp_path / "long", 41)
    reqs = rc.make_requests(cfg["vocab"], [900], seed=17)
    want = _oracle(model, reqs)
    scale = float(np.abs(want["r0"]).max())
    whole = _replay(model, None, torch.bfloat16, rc.whole(reqs), page_size=16)
    _compare(whole, want, reqs, scale, torch.bfloat16, "whole")
    cut = _replay(model, None, torch.bfloat16, rc.portions(reqs, (300, 129, 2, 270, 199)), page_size=16)
    _compare(cut, want, reqs, scale, torch.bfloat16, "portions")
    _compare(_replay(model, None, torch.float32, rc.whole(reqs), page_size=16), want, reqs, scale, torch.float32, "fp32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(von_dirs, cases, tmp_path, dtype):
    name = "von_c"
    reqs, want, scale = cases[name]
    steps = rc.mixed(reqs, seed=4)
    out_dir = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(von_dirs[name]), "--dtype", dtype,
         "--out", str(out_dir), "--max-tokens", str(rc.max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = tv.ALL[name]["vocab"]
    outs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
            for s in steps if any(e["want"] for e in s["entries"])}
    _compare(rc.collect(steps, outs), want, reqs, scale, torch.float32 if dtype == "float32" else torch.bfloat16,
             "trace_run")


@pytest.mark.parametrize("name", ["von_a", "von_b", "von_c"])
def test_greedy_generation_through_the_entry_point(von_dirs, name):
    from emberserve_b200 import LLM, SamplingParams

    cfg, w = plain.read_model_dir(von_dirs[name])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 5, 11, 30)]
    want = [plain.greedy(cfg, w, p, 10) for p in prompts]
    for how in (dict(), dict(max_num_batched_tokens=7), dict(enable_cuda_graphs=False, async_scheduling=False)):
        llm = LLM(str(von_dirs[name]), dtype="float32", device=DEV, block_size=tv.PAGE_SIZES[name],
                  num_gpu_blocks=256, max_model_len=128, max_num_seqs=3, **how)
        got = [r.output_token_ids for r in llm.generate(prompts, SamplingParams.greedy(10, ignore_eos=True))]
        assert got == want, how
        st = llm.engine.runner.cache.stats()
        assert st.num_free == st.num_pages


def test_command_line_random_weights_then_generate(tmp_path):
    """`random-weights` writes a Vonulix folder from its config.json; `generate` on it prints the tokens
    that LLM.generate returns (sampled with a seed, bfloat16, decode steps from CUDA graphs)."""
    from emberserve_b200 import LLM, SamplingParams

    (tmp_path / "config.json").write_text(json.dumps(VON_T))
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
