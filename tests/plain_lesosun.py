"""A plain, slow implementation of the Lesosun decoder: one function per mechanism, whole
sequences at once, token-by-token recurrences, dense masks, no cache and no batching.  It
shares no code with the package; the tests compare the engine with it.

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


# ---- small mechanisms ------------------------------------------------------------------

def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_erf(z):
    return 0.5 * z * (1 + torch.erf(z / math.sqrt(2.0)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def short_conv(u, taps_w, bias=None):
    """y[t] = sum_j w[:, j] u[t - taps + 1 + j] over time for every channel, zeros before t = 0.
    u: [T, C]; taps_w: [C, taps]."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat((torch.zeros(taps - 1, C, dtype=u.dtype), u))
    y = sum(taps_w[:, j] * padded[j:j + T] for j in range(taps))
    return y if bias is None else y + bias


def rotate_interleaved(x, dims, base):
    """x: [T, heads, D]; the pair (2i, 2i+1), i < dims / 2, of every head is turned by t * base^(-2i/dims)."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=x.dtype)
    ang = torch.arange(T, dtype=x.dtype)[:, None] * base ** (-2 * i / dims)  # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---- mixers ----------------------------------------------------------------------------

def capped_attention(h, w, p, m, eps):
    """Grouped-query attention: biased projections, a short convolution on q, k and v, a per-head RMS
    norm of q and k with a gain, a partial interleaved rotation, scores through a tanh cap, causal softmax."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"]).view(T, H, D)
    k = short_conv(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"]).view(T, G, D)
    v = short_conv(h @ w[p + "v"].T + w[p + "v.b"], w[p + "v.conv"]).view(T, G, V)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    if m.get("rot"):
        q = rotate_interleaved(q, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_interleaved(k, m["rot"]["dims"], m["rot"]["base"])
    out = torch.zeros(T, H, V, dtype=h.dtype)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        cap = m.get("softcap")
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~causal, -math.inf)
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * V) @ w[p + "o"].T + w[p + "o.b"]


def state_space(h, w, p, m, eps):
    """A selective state space per head with a scalar decay: S_t = exp(-exp(A) dt_t) S_(t-1) + dt_t B_t x_t^T,
    y_t = S_t^T C_t + D x_t; gated by silu(z), then normed in groups."""
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])  # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(N, V, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m["left_scale"] * capped_attention(h, w, p + "left.", m["left"], eps)
            + m["right_scale"] * state_space(h, w, p + "right.", m["right"], eps))


def channel_delta(h, w, p, m, eps):
    """The delta rule with a decay per key channel: S <- g S (rows), u = beta (v - S^T k), S <- S + k u^T,
    o = S^T q."""
    T = h.shape[0]
    H, K, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, K, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, K, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)  # [T, H]
    low = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(low).view(T, H, D))
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, V)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        kh = head // (H // K)
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = g[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            o[t, head] = S.T @ q[t, kh]
    o = rms(o, eps) * w[p + "norm"] * gate
    return o.reshape(T, H * V) @ w[p + "o"].T


MIXERS = {"parallel": parallel_mixer, "channel_delta": channel_delta}


# ---- feed-forwards ---------------------------------------------------------------------

def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def small_ff(h, up, down):
    return gelu_erf(h @ up.T) @ down.T


def routed_ff(h, w, p, mlp, choices_out=None):
    r = mlp["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)  # over E + I
    choice = s + w[p + "correction"] if (p + "correction") in w else s
    chosen = torch.topk(choice, top, dim=-1).indices  # [T, top]
    if choices_out is not None:
        choices_out.append((choice, chosen))
    picked = torch.gather(s, 1, chosen)
    weights = picked / (picked.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            y = h[t] if e >= E else small_ff(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
            out[t] += weights[t, j] * y
    if mlp.get("shared"):
        out = out + small_ff(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


def feed_forward(h, w, p, mlp):
    return dense_ff(h, w, p) if mlp["kind"] == "dense" else routed_ff(h, w, p, mlp)


# ---- the model -------------------------------------------------------------------------

def forward(cfg, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence; with `layers_out` (a list) the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = rms(x, eps) * (1 + w["embed.norm"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](rms(x, eps) * (1 + w[p + "norm1"]), w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(rms(x, eps) * (1 + w[p + "norm2"]), w, p + "mlp.", layer["mlp"])
        x = x + mult * y
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = (rms(x, eps) * (1 + w["final.norm"])) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
