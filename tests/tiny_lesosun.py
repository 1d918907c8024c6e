"""Tiny Lesosun configurations of the tests, and weights for them.

The three differ in every size and option: width, vocabulary, layer order (each mixer first, last and
twice in a row), layers without a feed-forward, query heads per key head (1, 2, 3), key and value sizes
that are equal and that differ, rotation of a few, of all and of no numbers of a head, with and without
a cap on the scores and on the logits, convolutions of 1 (no state), 2, 3 and 4 taps, state-space
groups and norm groups of 1 and more, delta heads that share q and k, inner sizes of the two-step
projections that are no multiples of 8, experts with and without identity experts and a shared expert,
one chosen expert and several, every weight of the sums different from 1 and equal to 1.

Weights are drawn wide (matrices of unit-order rows, gains around their centre, biases and decay
parameters of order 1) so that a wrong tap, pairing, gate, cap or decay moves the logits by far more
than any tolerance.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from emberserve_b200.config.lesosun import LesosunConfig
from emberserve_b200.weights.safetensors_io import write_safetensors


def _left(heads, kv_heads, dim, vdim, conv, rot_dims, base, softcap, scale=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
         "scale": scale if scale is not None else 1.7 / math.sqrt(dim)}
    if softcap:
        d["softcap"] = softcap
    if rot_dims:
        d["rot"] = {"base": base, "dims": rot_dims}
    return d


def _right(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def _parallel(left, right, mlp, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


def _delta(heads, kv_heads, dim, vdim, conv, ranks, mlp):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                               "conv": conv, "decay_rank": ranks[0], "gate_rank": ranks[1]}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, identity, top, scale, shared):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top,
                                                          "scale": scale}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


LES_A = {
    "architecture": "Lesosun", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "max_positions": 512,
    "residual_mult": 0.7, "logit_softcap": 12.0,
    "layers": [
        _delta(4, 2, 8, 12, 3, (5, 7), _dense(40)),
        _parallel(_left(6, 2, 8, 16, 2, 4, 100.0, 6.0), _right(4, 6, 5, 2, 2, 4), _moe(24, 5, 2, 2, 1.5, 16), 0.8, 1.2),
        _parallel(_left(2, 2, 16, 16, 1, 16, 10000.0, None), _right(3, 8, 8, 1, 1, 1), None, 1.0, 1.0),
    ],
}

LES_B = {
    "architecture": "Lesosun", "vocab": 130, "width": 64, "norm": {"eps": 3e-6}, "max_positions": 512,
    "residual_mult": 1.0,
    "layers": [
        _parallel(_left(3, 1, 24, 8, 4, 6, 50.0, 3.0, 0.3), _right(6, 4, 16, 3, 4, 2), _dense(72), 1.3, 0.6),
        _delta(2, 2, 16, 16, 1, (8, 3), _moe(16, 3, 0, 1, 1.0, None)),
        _delta(6, 1, 4, 40, 4, (2, 11), None),
        _parallel(_left(4, 4, 8, 24, 3, 0, 0.0, 9.0), _right(2, 20, 4, 2, 1, 3), _moe(8, 9, 3, 4, 2.5, 32), 0.5, 2.0),
    ],
}

LES_C = {
    "architecture": "Lesosun", "vocab": 61, "width": 40, "norm": {"eps": 1e-4}, "max_positions": 512,
    "residual_mult": 0.4, "logit_softcap": 5.0,
    "layers": [
        _delta(3, 3, 33, 70, 2, (9, 9), _moe(40, 4, 1, 5, 0.9, 8)),
        _delta(1, 1, 8, 8, 5, (4, 6), _dense(24)),
        _parallel(_left(5, 1, 8, 8, 5, 8, 7.0, 50.0), _right(1, 24, 33, 1, 3, 5), _dense(16), 1.0, 0.9),
    ],
}

ALL = {"les_a": LES_A, "les_b": LES_B, "les_c": LES_C}
SEEDS = {"les_a": 30, "les_b": 31, "les_c": 32}
PAGE_SIZES = {"les_a": 4, "les_b": 16, "les_c": 8}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    """Every tensor of a model of this design, by the names the checkpoint uses."""
    w = cfg["width"]
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg["vocab"], w), "embed.norm": (w,), "final.norm": (w,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        shapes[p + "norm1"] = (w,)
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            nq, nk, nv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"]
            shapes.update({q + "q": (nq, w), q + "q.b": (nq,), q + "k": (nk, w), q + "k.b": (nk,), q + "v": (nv, w),
                           q + "v.b": (nv,), q + "q.norm": (a["dim"],), q + "k.norm": (a["dim"],),
                           q + "q.conv": (nq, a["conv"]), q + "k.conv": (nk, a["conv"]), q + "v.conv": (nv, a["conv"]),
                           q + "o": (w, a["heads"] * a["vdim"]), q + "o.b": (w,)})
            q = p + "mix.right."
            inner, gn, h = r["heads"] * r["vdim"], r["groups"] * r["state"], r["heads"]
            shapes.update({q + "in": (2 * inner + 2 * gn + h, w), q + "conv": (inner + 2 * gn, r["conv"]),
                           q + "conv.b": (inner + 2 * gn,), q + "dt_bias": (h,), q + "A_log": (h,), q + "D": (h,),
                           q + "norm": (inner,), q + "o": (w, inner)})
        else:
            q = p + "mix."
            nk, nv, h = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"]
            shapes.update({q + "q": (nk, w), q + "q.conv": (nk, m["conv"]), q + "k": (nk, w), q + "k.conv": (nk, m["conv"]),
                           q + "v": (nv, w), q + "v.conv": (nv, m["conv"]), q + "b": (h, w), q + "A_log": (h,),
                           q + "norm": (m["vdim"],), q + "a1": (m["decay_rank"], w), q + "a2": (h * m["dim"], m["decay_rank"]),
                           q + "dt_bias": (h * m["dim"],), q + "g1": (m["gate_rank"], w),
                           q + "g2": (nv, m["gate_rank"]), q + "o": (w, nv)})
        f = L.get("mlp")
        if f is None:
            continue
        shapes[p + "norm2"] = (w,)
        q = p + "mlp."
        if f["kind"] == "dense":
            shapes.update({q + "gate": (f["ff"], w), q + "up": (f["ff"], w), q + "down": (w, f["ff"])})
        else:
            r = f["router"]
            total = r["experts"] + r.get("identity", 0)
            shapes.update({q + "router": (total, w), q + "correction": (total,)})
            for e in range(r["experts"]):
                shapes.update({f"{q}e{e}.up": (f["expert"]["ff"], w), f"{q}e{e}.down": (w, f["expert"]["ff"])})
            if f.get("shared"):
                shapes.update({q + "shared.up": (f["shared"]["ff"], w), q + "shared.down": (w, f["shared"]["ff"])})
    return shapes


def make_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("q.norm", "k.norm", "mix.norm", "right.norm")):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)  # plain gains
        elif last in ("norm", "norm1", "norm2"):
            t = 0.3 * torch.randn(shape, generator=gen)  # gains stored minus one
        elif last == "conv":
            t = 0.7 * torch.randn(shape, generator=gen)
        elif last == "A_log":
            t = -0.5 + 0.7 * torch.randn(shape, generator=gen)
        elif last == "dt_bias":
            t = -1.0 + torch.randn(shape, generator=gen)
        elif last == "D":
            t = 1.0 + 0.5 * torch.randn(shape, generator=gen)
        elif last == "correction":
            t = 0.1 * torch.randn(shape, generator=gen)
        elif last == "b" and len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) * (1.5 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(cfg: dict, out_dir, seed: int, weights: dict[str, torch.Tensor] | None = None) -> Path:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(out / "model.safetensors", weights if weights is not None else make_weights(cfg, seed))
    return out


def typed(cfg: dict) -> LesosunConfig:
    return LesosunConfig.from_dict(cfg)
