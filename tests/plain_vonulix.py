"""A plain, slow implementation of the Vonulix decoder: one function per mechanism, whole
sequences at once, dense masks, no cache and no batching.  It shares no code with the
package; the tests compare the engine with it.

Notation: a sequence is ``x[t, :]`` with positions t = 0, 1, ...; weights are ``[out, in]``
and act as ``x @ W.T``.  Everything is computed in the dtype the tensors are given in
(the tests use float64).
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ---- reading a model folder ------------------------------------------------------------

def read_safetensors(path) -> dict[str, torch.Tensor]:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = np.frombuffer(data[lo:hi], dtype=np.uint8)
        kind = info["dtype"]
        if kind == "BF16":
            u = buf.view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif kind == "F32":
            t = torch.from_numpy(buf.view(np.float32).copy())
        elif kind == "I32":
            t = torch.from_numpy(buf.view(np.int32).copy())
        else:
            raise ValueError(kind)
        out[name] = t.reshape(info["shape"])
    return out


def read_model_dir(model_dir):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    return cfg, read_safetensors(model_dir / "model.safetensors")


# ---- mechanisms ------------------------------------------------------------------------

def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the gain minus one."""
    return unit_rms(x, eps) * (1 + w)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def turn_halves(x, angles):
    """x: [T, heads, n]; angles: [T, r/2].  Number i of the first r is paired with number i + r/2 and
    the pair is turned by angles[t, i]; what lies past r is left alone."""
    half = angles.shape[1]
    c, s = torch.cos(angles)[:, None, :], torch.sin(angles)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def pair_frequencies(n, base, dtype):
    """base^(-2i/n) for the n/2 pairs of n numbers."""
    return base ** (-2 * torch.arange(n // 2, dtype=dtype) / n)


def visible(T, size, keep_first):
    """[T, T] bool: query i sees key j iff j <= i and (i - j < size or j < keep_first)."""
    t = torch.arange(T)
    i, j = t[:, None], t[None, :]
    near = (i - j < size) if size else torch.ones(T, T, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def attention(h, w, p, m, eps):
    """Grouped-query attention: rotary on the first numbers of every q and k head with all
    frequencies divided by a factor; values unit-normed per head and turned by their own position
    over their whole length, the sum over values turned back by the query's position; a window
    that also keeps the first tokens; a sigmoid gate per head before the output projection."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    pos = torch.arange(T, dtype=h.dtype)
    rot = m["rot"]
    f = pair_frequencies(rot["dims"], rot["base"], h.dtype) / ((rot.get("scaling") or {}).get("factor", 1.0))
    ang = pos[:, None] * f[None, :]
    q, k = turn_halves(q, ang), turn_halves(k, ang)
    v = unit_rms(v, eps)
    vang = pos[:, None] * pair_frequencies(V, rot["base"], h.dtype)[None, :]
    v = turn_halves(v, vang)
    mask = m.get("mask") or {}
    seen = visible(T, mask.get("size"), mask.get("keep_first", 0))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, -math.inf)
        out[:, head] = torch.softmax(s, -1) @ v[:, g]
    out = turn_halves(out, -vang)
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].T


def capped_expert(h, gate, up, down, limit):
    """g = min(Wg h, limit); u = clamp(Wu h, -limit, limit); Wd (g sigmoid(1.702 g) (u + 1))."""
    g = (h @ gate.T).clamp(max=limit)
    u = (h @ up.T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ down.T


def routed_experts(h, w, p, m):
    """Sigmoid scores, the `top` largest chosen, the score multiplies the expert's INPUT; a shared
    expert for every token, times one sigmoid number per token."""
    T = h.shape[0]
    E, top = m["router"]["experts"], m["router"]["top"]
    limit = m["expert"]["limit"]
    s = torch.sigmoid(h @ w[p + "router"].T)  # [T, E]
    out = torch.zeros(T, w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            q = f"{p}e{e}."
            out[t] += capped_expert(s[t, e] * h[t], w[q + "gate"], w[q + "up"], w[q + "down"], limit)
    sh = m.get("shared")
    if sh:
        q = p + "shared."
        y = capped_expert(h, w[q + "gate"], w[q + "up"], w[q + "down"], sh["limit"])
        out = out + torch.sigmoid(h @ w[q + "sg"].T) * y
    return out


def token_side_input(x, tokens, w, layer, dim, eps):
    """What a layer adds from the token's own row of a second table."""
    p = f"l{layer}.side."
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    y = g @ w[p + "proj"].T
    return unit_rms(y, eps) * w[p + "norm"]


def forward(cfg, w, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one sequence.  `streams`, a list, receives each layer's result."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    history = [x]
    side = cfg.get("token_side")
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert L["type"] == "attention"
        x = x + attention(offset_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            x = x + routed_experts(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.", L["mlp"])
        if side:
            x = x + token_side_input(x, tokens, w, i, side["dim"], eps)
        if streams is not None:
            streams.append(x)
        history.append(x)
        if p + "dwa" in w:
            x = sum(w[p + "dwa"][j] * history[j] for j in range(i + 2))
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg, w, prompt, count, dtype=torch.float64):
    """`count` tokens generated greedily behind `prompt` (the whole sequence is recomputed each time)."""
    seq = list(prompt)
    for _ in range(count):
        seq.append(int(forward(cfg, w, seq, dtype)[-1].argmax()))
    return seq[len(prompt):]
