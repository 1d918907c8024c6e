"""Tiny Vonulix configurations of the tests, and weights for them.

The three differ in every size and option: width, vocabulary, number of layers, layers without a
feed-forward, query heads per key head (1, 3, 5), key and value heads of unequal size (either one the
larger), windows of 1, of a few keys (no multiple of a page) and none at all, kept first keys from
none to more than the window, rotation of a few or of all numbers of a head, with and without linear
scaling, one to three chosen experts of 3 to 9, with and without a shared expert (of another size and
limit than the routed ones), with and without the per-layer token input, embedding scales and eps.

Weights are drawn wide (matrices of unit-order rows, norm weights around zero, gains around one,
depth weights of order one) so that a wrong pair, window edge, expert, weight or depth moves the
logits by far more than any tolerance.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from emberserve_b200.config.vonulix import VonulixConfig
from emberserve_b200.weights.safetensors_io import write_safetensors


def _mixer(heads, kv_heads, dim, vdim, window, keep, rot_dims, base, factor=None, scale=None):
    d = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else 1.7 / math.sqrt(dim), "rot": {"base": base, "dims": rot_dims}}
    if factor is not None:
        d["rot"]["scaling"] = {"factor": factor}
    if window is not None or keep:
        d["mask"] = {"size": window, "keep_first": keep}
    return d


def _moe(experts, top, ff, limit, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        d["shared"] = {"ff": shared[0], "limit": shared[1]}
    return d


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


VON_A = {
    "architecture": "Vonulix", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "max_positions": 512,
    "embedding": {"scale": 3.5}, "token_side": {"dim": 4},
    "layers": [
        _layer(_mixer(6, 2, 8, 16, 7, 3, 4, 100.0, 2.0), _moe(5, 2, 24, 1.5, (40, 0.8))),
        _layer(_mixer(3, 3, 16, 8, 5, 0, 16, 1000.0), None),
        _layer(_mixer(6, 2, 8, 16, 7, 3, 4, 100.0, 2.0), _moe(5, 2, 24, 1.5, (40, 0.8))),
    ],
}

VON_B = {
    "architecture": "Vonulix", "vocab": 130, "width": 64, "norm": {"eps": 3e-6}, "max_positions": 512,
    "embedding": {"scale": 1.0},
    "layers": [
        _layer(_mixer(4, 4, 16, 8, 40, 0, 16, 10000.0), _moe(3, 3, 32, 2.5)),
        _layer(_mixer(2, 1, 24, 32, None, 0, 6, 50.0, 8.0, 0.3), _moe(4, 1, 16, 1.0, (16, 3.0))),
        _layer(_mixer(4, 4, 16, 8, 40, 11, 16, 10000.0), _moe(3, 3, 32, 2.5)),
        _layer(_mixer(8, 2, 8, 8, 16, 16, 2, 7.0, 1.5), None),
    ],
}

VON_C = {
    "architecture": "Vonulix", "vocab": 61, "width": 40, "norm": {"eps": 1e-4}, "max_positions": 512,
    "embedding": {"scale": 0.6}, "token_side": {"dim": 9},
    "layers": [
        _layer(_mixer(5, 1, 24, 24, 1, 9, 24, 500.0, 3.0), _moe(9, 1, 8, 0.7, (24, 2.0))),
        _layer(_mixer(5, 5, 8, 40, 130, 2, 8, 20.0), _moe(6, 4, 12, 4.0)),
    ],
}

ALL = {"von_a": VON_A, "von_b": VON_B, "von_c": VON_C}
SEEDS = {"von_a": 30, "von_b": 31, "von_c": 32}
PAGE_SIZES = {"von_a": 4, "von_b": 16, "von_c": 8}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    """Every tensor of a model of this design, by the names the checkpoint uses."""
    w = cfg["width"]
    side = (cfg.get("token_side") or {}).get("dim", 0)
    shapes: dict[str, tuple[int, ...]] = {"embed": (cfg["vocab"], w), "head": (cfg["vocab"], w), "final.norm": (w,)}
    if side:
        shapes["side.embed"] = (cfg["vocab"], side * len(cfg["layers"]))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        q = p + "mix."
        shapes.update({p + "norm1": (w,), q + "q": (m["heads"] * m["dim"], w), q + "k": (m["kv_heads"] * m["dim"], w),
                       q + "v": (m["kv_heads"] * m["vdim"], w), q + "g": (m["heads"], w),
                       q + "o": (w, m["heads"] * m["vdim"]), p + "dwa": (i + 2,)})
        mlp = L.get("mlp")
        if mlp is not None:
            q, ff = p + "mlp.", mlp["expert"]["ff"]
            shapes.update({p + "norm2": (w,), q + "router": (mlp["router"]["experts"], w)})
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{q}e{e}.gate": (ff, w), f"{q}e{e}.up": (ff, w), f"{q}e{e}.down": (w, ff)})
            if mlp.get("shared"):
                ff = mlp["shared"]["ff"]
                shapes.update({q + "shared.gate": (ff, w), q + "shared.up": (ff, w), q + "shared.down": (w, ff),
                               q + "shared.sg": (1, w)})
        if side:
            shapes.update({p + "side.gate": (side, w), p + "side.proj": (w, side), p + "side.norm": (w,)})
    return shapes


def make_weights(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        last = name.rsplit(".", 1)[-1]
        if name.endswith("side.norm"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)  # a plain gain
        elif last in ("norm", "norm1", "norm2"):
            t = 0.3 * torch.randn(shape, generator=gen)  # stored around zero
        elif last == "dwa":
            t = 0.5 * torch.randn(shape, generator=gen)
            t[-1] += 1.0
        elif name in ("embed", "side.embed"):
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


def typed(cfg: dict) -> VonulixConfig:
    return VonulixConfig.from_dict(cfg)
