"""Plain PyTorch restatements of every kernel of ``emberserve_b200.kernels``: same
arguments, same effects, 32-bit (or 64-bit) arithmetic, loops where loops are clearest.

Two uses: the GPU tests compare each CUDA kernel with its restatement here, and the
host-logic tests (no GPU) swap these in for the kernels so that the step function, the
cache and the replay tool can be exercised on the CPU.  Nothing in the package imports
this file.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def embedding(table, tokens, residual, deferred=None, scale=1.0):
    n = residual.shape[0]
    tok = tokens[:n].long()
    if deferred is not None and bool((tok < 0).any()):
        tok = torch.where(tok < 0, deferred.long()[(-(tok + 1)).clamp(min=0)], tok)
    residual.copy_(table[tok].float() * torch.tensor(scale, dtype=torch.float32))


def add_rmsnorm(delta, residual, weight, out, eps, rows=None, num_rows=None):
    if rows is None:
        r = residual if delta is None else residual + delta[:residual.shape[0]].float()
        if delta is not None:
            residual.copy_(r)
    else:
        idx = rows[: (rows.numel() if num_rows is None else num_rows)].long()
        r = residual[idx]
        if delta is not None:
            r = r + delta[idx].float()
    y = (r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps)).to(out.dtype).float()
    out[: r.shape[0]].copy_((y * weight.float()).to(out.dtype))


def silu_mul(gate_up, out):
    i = out.shape[1]
    g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def rope_table(inv_freq, max_pos):
    ang = torch.arange(max_pos, dtype=torch.float32, device=inv_freq.device)[:, None] * inv_freq[None, :]
    return torch.stack((ang.cos(), ang.sin()), dim=-1).contiguous()


def _rotate(x, cs, rot):
    """x: [N, heads, D] float; cs: [N, rot/2, 2]."""
    half = rot // 2
    c, s = cs[:, None, :, 0], cs[:, None, :, 1]
    x1, x2 = x[..., :half], x[..., half:rot]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]), dim=-1)


def rope_kv_write(qkv, num_heads, num_kv_heads, head_dim, positions, row_of_token, table, rotary_dim,
                  kcache, vcache, block_tables, page_size, write_kv=True):
    n = qkv.shape[0]
    d = head_dim
    q = qkv[:, : num_heads * d].float().view(n, num_heads, d)
    k = qkv[:, num_heads * d:(num_heads + num_kv_heads) * d].float().view(n, num_kv_heads, d)
    v = qkv[:, (num_heads + num_kv_heads) * d:].view(n, num_kv_heads, d)
    pos = positions[:n].long()
    if rotary_dim > 0:
        cs = table[pos]
        q = _rotate(q, cs, rotary_dim)
        k = _rotate(k, cs, rotary_dim)
    qkv[:, : num_heads * d] = q.reshape(n, -1).to(qkv.dtype)
    if not write_kv:
        return
    rows = row_of_token[:n].long()
    page = block_tables[rows, pos // page_size].long()
    slot = pos % page_size
    kcache[page, :, slot, :] = k.to(kcache.dtype)
    vcache[page, :, slot, :] = v.to(vcache.dtype)


def attention_scratch_bytes(num_tokens, num_heads, head_dim, splits):
    return 0 if splits <= 1 else num_tokens * num_heads * splits * (head_dim + 2) * 4


def paged_attention(q, out, kcache, vcache, block_tables, cu_q, starts, num_rows, num_tokens,
                    num_heads, num_kv_heads, head_dim, scale, max_q_len, window=None, splits=1,
                    scratch=None, generic=False, tcgen05=False, kernel="auto", compute_dtype=torch.float32):
    """Per request: gather its keys and values from the pages, dense masked softmax."""
    page_size = kcache.shape[2]
    groups = num_heads // num_kv_heads
    cu = cu_q.tolist()
    st = starts.tolist()
    for b in range(num_rows):
        q0, q1 = cu[b], cu[b + 1]
        qlen, ctx = q1 - q0, st[b] + (q1 - q0)
        if qlen == 0:
            continue
        lo = 0 if not window else max(0, st[b] - window + 1)
        keys = torch.arange(lo, ctx, device=q.device)
        pages = block_tables[b, keys // page_size].long()
        k = kcache[pages, :, keys % page_size, :].to(compute_dtype)  # [T, Hkv, D]
        v = vcache[pages, :, keys % page_size, :].to(compute_dtype)
        qq = q[q0:q1, : num_heads * head_dim].to(compute_dtype).view(qlen, num_heads, head_dim)
        kf = k.repeat_interleave(groups, dim=1).permute(1, 0, 2)
        vf = v.repeat_interleave(groups, dim=1).permute(1, 0, 2)
        scores = torch.matmul(qq.permute(1, 0, 2), kf.transpose(-1, -2)) * scale  # [H, qlen, T]
        qpos = torch.arange(st[b], ctx, device=q.device)[:, None]
        hidden = keys[None, :] > qpos
        if window:
            hidden = hidden | (keys[None, :] <= qpos - window)
        scores = scores.masked_fill(hidden, float("-inf"))
        o = torch.matmul(torch.softmax(scores, dim=-1), vf).permute(1, 0, 2)
        out[q0:q1] = o.reshape(qlen, num_heads * head_dim).to(out.dtype)


def argmax(logits, out):
    out[: logits.shape[0]].copy_(torch.argmax(logits, dim=-1).to(torch.int32))


@torch.inference_mode()  # the logits of a step are inference tensors
def repetition_penalty(logits, row_ptr, token_ids, penalty):
    ptr = row_ptr.tolist()
    for r in range(logits.shape[0]):
        p = float(penalty[r])
        if p == 1.0:
            continue
        for tok in sorted(set(token_ids[ptr[r]:ptr[r + 1]].tolist())):
            s = float(logits[r, tok])
            logits[r, tok] = s / p if s > 0 else s * p


# ---- sampling: Philox4x32-10 and the draw, restated with numpy ----------------------------

def philox4x32_10(key: tuple[int, int], ctr: tuple[int, int, int, int]) -> tuple[int, int, int, int]:
    m0, m1, w0, w1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    k0, k1 = key
    c0, c1, c2, c3 = ctr
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c3 ^ k1) & mask, p0 & mask
        k0, k1 = (k0 + w0) & mask, (k1 + w1) & mask
    return c0, c1, c2, c3


def uniform_of(seed: int, counter: int) -> float:
    seed &= 0xFFFFFFFFFFFFFFFF
    counter &= 0xFFFFFFFFFFFFFFFF
    x = philox4x32_10((seed & 0xFFFFFFFF, seed >> 32), (counter & 0xFFFFFFFF, counter >> 32, 0, 0))[0]
    return float(np.float32(x >> 8) * np.float32(1.0 / 16777216.0))


def kept_mask(z: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    """Which tokens survive top-k then top-p (emberserve/sampling.py:56-73), z = logits / T."""
    v = z.numel()
    keep = torch.ones(v, dtype=torch.bool)
    if 0 < top_k < v:
        keep &= z >= torch.topk(z, top_k).values[-1]
    if top_p < 1.0:
        zz = z.masked_fill(~keep, float("-inf")).double()
        probs = torch.softmax(zz, dim=-1)
        order = torch.argsort(zz, descending=True, stable=True)
        sp = probs[order]
        # mass strictly above a token = mass of all tokens with a larger value
        mass_before = torch.zeros(v, dtype=torch.float64)
        csum = torch.cumsum(sp, 0) - sp
        sv = zz[order]
        first_of_value = torch.ones(v, dtype=torch.bool)
        first_of_value[1:] = sv[1:] != sv[:-1]
        idx_first = torch.cummax(torch.where(first_of_value, torch.arange(v), torch.zeros(v, dtype=torch.long)), 0).values
        mass_before[order] = csum[idx_first]
        keep &= mass_before < top_p
    return keep


def sample(logits, temperature, top_k, top_p, seeds, counters, out):
    """Token per row: argmax where temperature == 0, else inverse-CDF draw with the
    Philox uniform, in index order over the kept tokens (32-bit sums, as the kernel)."""
    for r in range(logits.shape[0]):
        x = logits[r].float().cpu()
        t = float(temperature[r])
        if t == 0.0:
            out[r] = int(torch.argmax(x))
            continue
        z = x / np.float32(t)
        keep = kept_mask(z, int(top_k[r]), float(top_p[r]))
        e = torch.where(keep, torch.exp(z - z.max()), torch.zeros_like(z)).double()
        u = uniform_of(int(seeds[r]), int(counters[r]))
        c = torch.cumsum(e, 0)
        target = u * float(c[-1])
        idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64), right=True))
        kept_idx = torch.nonzero(keep).flatten()
        idx = min(idx, int(kept_idx[-1]))
        out[r] = idx


GEMM_SMALLM_MAX_ROWS = 64


def gemm_smallm(x, weight, bias, out, ksplit=1):
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    out.copy_(y.to(out.dtype))


def gemm_smallm_gated(x, weight, out):
    i = out.shape[1]
    y = x.float() @ weight.float().t()
    g, u = y[:, :i], y[:, i:]
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def check_status(clear=True):
    return None


# ---- the residual stream of decoders with a norm on both sides of every sub-layer ----------

def stream_inject(residual, tokens, embed, table, row=0, deferred=None):
    n = residual.shape[0]
    if embed is not None:
        tok = tokens[:n].long()
        if deferred is not None and bool((tok < 0).any()):
            tok = torch.where(tok < 0, deferred.long()[(-(tok + 1)).clamp(min=0)], tok)
        residual += embed[tok].float()
    if table is not None:
        residual += table[row].float()


def _group_norm(x, groups, eps):
    n, h = x.shape
    parts = x.view(n, groups, h // groups)
    return (parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, h)


def add_norm_grouped(delta, post_gain, post_groups, post_eps, residual, gain, groups, eps, out, rows=None):
    idx = None if rows is None else rows.long()
    r = residual if idx is None else residual[idx]
    if delta is not None:
        d = (delta[:residual.shape[0]] if idx is None else delta[idx]).float()
        if post_gain is not None:
            d = _group_norm(d, post_groups, post_eps) * post_gain.float()
        r = r + d
        if idx is None:
            residual.copy_(r)
    out[:r.shape[0]].copy_((_group_norm(r, groups, eps) * gain.float()).to(out.dtype))


def _glu_activation(g, act):
    if act == "relu":
        return torch.relu(g)
    if act == "gelu_tanh":
        return 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    return g / (1 + torch.exp(-g))


def _glu(g, u, act, limit, alpha):
    if act == "swiglu_capped":
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
        return g * torch.sigmoid(alpha * g) * (u + 1)
    return _glu_activation(g, act) * u


def glu_act(gate_up, out, act, limit=0.0, alpha=1.0, row_gate=False):
    i = out.shape[1]
    g, u = gate_up[:, :i].float(), gate_up[:, i:2 * i].float()
    y = _glu(g, u, act, limit, alpha)
    if row_gate:
        y = y * torch.sigmoid(gate_up[:, 2 * i].float())[:, None]
    out.copy_(y.to(out.dtype))


def add_cast(delta, residual, out):
    if delta is not None:
        residual += delta[:residual.shape[0]].float()
    out.copy_(residual.to(out.dtype))


def token_gate(z, table, col0, tokens, out, deferred=None):
    n, c = z.shape
    tok = tokens[:n].long()
    if deferred is not None and bool((tok < 0).any()):
        tok = torch.where(tok < 0, deferred.long()[(-(tok + 1)).clamp(min=0)], tok)
    v = z.float()
    g = 0.5 * v * (1 + torch.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    out.copy_((g * table[tok, col0:col0 + c].float()).to(out.dtype))


def depth_mix(delta, gain, eps, residual, hist, weights, count):
    n = residual.shape[0]
    x = residual
    if delta is not None:
        d = delta[:n].float()
        if gain is not None:
            d = d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * gain.float()
        x = residual + d
    hist[count - 1].copy_(x)
    if weights is not None:
        x = sum(weights[j] * hist[j] for j in range(count))
    residual.copy_(x)


def causal_taps(x, weight, state, slots, cu_q, row_of_token, out, num_rows, bias=None, identity=True):
    taps = weight.shape[1]
    cu = cu_q.tolist()
    w = weight.float()
    for b in range(num_rows):
        q0, q1 = cu[b], cu[b + 1]
        if q1 <= q0:
            continue
        h = x[q0:q1].float()
        if taps > 1:
            slot = int(slots[b])
            full = torch.cat((state[slot], h), 0)
        else:
            full = h
        conv = torch.zeros_like(h)
        for j in range(taps):
            conv += w[:, j] * full[j:j + h.shape[0]]
        if bias is not None:
            conv = conv + bias.float()
        out[q0:q1] = ((h + conv) if identity else conv).to(out.dtype)
        if taps > 1:
            state[slot] = full[-(taps - 1):]


def _rotate_pairs(v, cs, dims, pairing):
    """v: [..., >= dims] float; cs: [..., dims/2, 2] broadcastable."""
    half = dims // 2
    c, s = cs[..., 0], cs[..., 1]
    out = v.clone()
    if pairing == "half":
        a, b = v[..., :half], v[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    else:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


def latent_prep(proj, q_rank, kv_rank, rope_dim, q_gain, kv_gain, eps, positions, row_of_token, table, rot_dims,
                pairing, pages, block_tables, cq, write=True):
    n = proj.shape[0]
    p = proj.float()
    ql = p[:, :q_rank]
    cq.copy_((ql / torch.sqrt(ql.pow(2).mean(-1, keepdim=True) + eps) * q_gain.float()).to(cq.dtype))
    if not write:
        return
    kv = p[:, q_rank:q_rank + kv_rank]
    c = kv / torch.sqrt(kv.pow(2).mean(-1, keepdim=True) + eps) * kv_gain.float()
    kr = p[:, q_rank + kv_rank:q_rank + kv_rank + rope_dim]
    pos = positions[:n].long()
    if rot_dims:
        kr = _rotate_pairs(kr, table[pos], rot_dims, pairing)
    page_size = pages.shape[1]
    page = block_tables[row_of_token[:n].long(), pos // page_size].long()
    pages[page, pos % page_size] = torch.cat((c, kr), -1).to(pages.dtype)


def rope_inplace(x, num_heads, head_stride, offset, rot_dims, pairing, positions, table):
    n = x.shape[0]
    cs = table[positions[:n].long()]
    for h in range(num_heads):
        lo = h * head_stride + offset
        v = x[:, lo:lo + rot_dims].float()
        x[:, lo:lo + rot_dims] = _rotate_pairs(v, cs, rot_dims, pairing).to(x.dtype)


def latent_attention_scratch_bytes(num_tokens, num_heads, kv_rank, splits):
    return 0 if splits <= 1 else num_tokens * num_heads * splits * (kv_rank + 2) * 4


def latent_attention(qlat, q, rot_offset, head_stride, pages, block_tables, positions, row_of_token, out,
                     num_heads, kv_rank, rope_dim, scale, splits=1, scratch=None, kernel="auto"):
    h, n, r = qlat.shape
    page_size = pages.shape[1]
    for t in range(n):
        pos, row = int(positions[t]), int(row_of_token[t])
        keys = torch.arange(pos + 1)
        vec = pages[block_tables[row, keys // page_size].long(), keys % page_size].float()  # [T, R + P]
        qr = q[t].float().view(num_heads, head_stride)[:, rot_offset:rot_offset + rope_dim]
        full = torch.cat((qlat[:, t].float(), qr), -1)  # [H, R + P]
        w = torch.softmax(full @ vec.t() * scale, -1)
        out[:, t] = (w @ vec[:, :kv_rank]).to(out.dtype)


def heads_gate(ov, gate, out):
    h, n, v = ov.shape
    y = ov.float().permute(1, 0, 2).reshape(n, h * v)
    if gate is not None:
        y = y / (1 + torch.exp(-gate.float()))
    out.copy_(y.to(out.dtype))


def moe_tile_rows():
    return 64


def moe_max_tiles(num_pairs, num_experts, tile_rows):
    return num_pairs // tile_rows + min(num_experts, num_pairs)


def moe_route(logits, top, renormalize, ids, weights, offsets, perm, plan, max_tiles, align=1, big=None, inv=None,
              scoring="softmax", correction=None, renorm_eps=0.0, scale=1.0, plan_experts=None):
    assert align == 1, "the aligned layout belongs to the GPU path"
    n, e = logits.shape
    s = torch.sigmoid(logits.float()) if scoring == "sigmoid" else torch.softmax(logits.float(), -1)
    chosen = torch.zeros(n, top, dtype=torch.long)
    z = logits.clone() if correction is None else s + correction.float()
    for k in range(top):
        chosen[:, k] = torch.argmax(z, -1)  # the first of equal maxima
        z[torch.arange(n), chosen[:, k]] = float("-inf")
    w = torch.gather(s, 1, chosen)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + renorm_eps)
    w = w * scale
    ids.view(-1)[:n * top] = chosen.reshape(-1).to(torch.int32)
    weights.view(-1)[:n * top] = w.reshape(-1)
    flat = chosen.reshape(-1)
    order = torch.argsort(flat, stable=True)
    perm[:n * top] = order.to(torch.int32)
    counts = torch.bincount(flat, minlength=e)
    offsets[0] = 0
    offsets[1:e + 1] = torch.cumsum(counts, 0).to(torch.int32)


def moe_up(x, wgu, perm, offsets, plan, max_tiles, top, act, out, kernel="auto", in_scale=None, limit=0.0,
           alpha=1.0, gated=True):
    e, ff2, k = wgu.shape
    ff = ff2 // 2
    off = offsets.tolist()
    if not gated:  # experts without a gate: act(x Wu^T) of the rounded sum
        for ex in range(e):
            lo, hi = off[ex], off[ex + 1]
            if hi > lo:
                y = x[(perm[lo:hi] // top).long()].float() @ wgu[ex].float().t()
                if in_scale is not None:
                    y = y * in_scale[perm[lo:hi].long()][:, None]
                y = y.to(out.dtype).float()
                if act == "gelu":
                    y = 0.5 * y * (1 + torch.erf(y / math.sqrt(2.0)))
                else:
                    y = _glu_activation(y, act)
                out[lo:hi] = y.to(out.dtype)
        return
    for ex in range(e):
        lo, hi = off[ex], off[ex + 1]
        if hi <= lo:
            continue
        rows = x[(perm[lo:hi] // top).long()].float()
        y = rows @ wgu[ex].float().t()
        if in_scale is not None:
            y = y * in_scale[perm[lo:hi].long()][:, None]
        if act != "swiglu_capped":  # (that one works on the unrounded sums)
            y = y.to(out.dtype).float()
        out[lo:hi] = _glu(y[:, :ff], y[:, ff:], act, limit, alpha).to(out.dtype)


def moe_down(act, wdown, perm, offsets, plan, max_tiles, y, kernel="auto"):
    e = wdown.shape[0]
    off = offsets.tolist()
    for ex in range(e):
        lo, hi = off[ex], off[ex + 1]
        if hi <= lo:
            continue
        y[perm[lo:hi].long()] = (act[lo:hi].float() @ wdown[ex].float().t()).to(act.dtype).float()


def moe_combine(y, weights, out, top, extra=None, ids=None, x=None, num_real=0):
    n, h = out.shape
    rows = y[:n * top].view(n, top, h)
    if x is not None:  # an expert at or past num_real returns its input
        same = ids.view(-1)[:n * top].view(n, top) >= num_real
        rows = torch.where(same[:, :, None], x.float()[:, None, :], rows)
    if weights is not None:
        rows = rows * weights.view(-1)[:n * top].view(n, top, 1)
    total = rows.sum(1)
    if extra is not None:
        total = total + extra.float()
    out.copy_(total.to(out.dtype))


def unary_act(x, out, act):
    z = x.float()
    if act == "relu":
        y = torch.relu(z)
    elif act == "relu2":
        y = torch.relu(z) ** 2
    elif act == "gelu_tanh":
        y = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    elif act == "gelu":
        y = 0.5 * z * (1 + torch.erf(z / math.sqrt(2.0)))
    else:
        y = z / (1 + torch.exp(-z))
    out.copy_(y.to(out.dtype))


def qk_prep(proj, num_heads, num_kv_heads, head_dim, positions, row_of_token, table, rot_dims, pairing, norm_eps,
            kcache, vcache, block_tables, values_are_keys, write=True, v_norm_eps=None, v_table=None,
            v_pairing="half", q_gain=None, k_gain=None, norm_first=False):
    n, d, dv = proj.shape[0], head_dim, vcache.shape[3]
    nq, nk = num_heads * d, num_kv_heads * d
    pos = positions[:n].long()
    q = proj[:, :nq].float().view(n, num_heads, d).clone()
    k_raw = proj[:, nq:nq + nk]
    k = k_raw.float().view(n, num_kv_heads, d)
    v = k_raw if values_are_keys else proj[:, nq + nk:nq + nk + num_kv_heads * dv]
    def normed(q, k):
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + norm_eps)
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + norm_eps)
        if q_gain is not None:
            q, k = q * q_gain.float(), k * k_gain.float()
        return q, k

    if norm_eps is not None and norm_first:
        q, k = normed(q, k)
    if table is not None and rot_dims:
        cs = table[pos][:, None]
        q, k = _rotate_pairs(q, cs, rot_dims, pairing), _rotate_pairs(k, cs, rot_dims, pairing)
    if norm_eps is not None and not norm_first:
        q, k = normed(q, k)
    vv = v.reshape(n, num_kv_heads, dv).clone()
    if v_norm_eps is not None or v_table is not None:
        vf = vv.float()
        if v_norm_eps is not None:
            vf = vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + v_norm_eps)
        if v_table is not None:
            vf = _rotate_pairs(vf, v_table[pos][:, None], dv, v_pairing)
        vv = vf
    proj[:, :nq] = q.reshape(n, nq).to(proj.dtype)
    if not write:
        return
    page_size = kcache.shape[2]
    page = block_tables[row_of_token[:n].long(), pos // page_size].long()
    kcache[page, :, pos % page_size, :] = k.to(kcache.dtype)
    vcache[page, :, pos % page_size, :] = vv.to(vcache.dtype)


def paged_attention_masked(q, out, kcache, vcache, block_tables, cu_q, starts, num_rows, num_tokens, num_heads,
                           num_kv_heads, head_dim, scale, max_q_len, window=None, chunk=None, sinks=None, gate=None,
                           splits=1, scratch=None, kernel="auto", keep_first=0, out_table=None, out_pairing="half",
                           positions=None, softcap=None):
    page_size = kcache.shape[2]
    dv = vcache.shape[3]
    groups = num_heads // num_kv_heads
    cu, st = cu_q.tolist(), starts.tolist()
    for b in range(num_rows):
        q0, q1 = cu[b], cu[b + 1]
        qlen, ctx = q1 - q0, st[b] + (q1 - q0)
        if qlen == 0:
            continue
        lo = 0
        if window:
            lo = max(lo, st[b] - window + 1)
        if chunk:
            lo = max(lo, (st[b] // chunk) * chunk)
        kept = min(keep_first or 0, lo) if (window or chunk) else 0
        keys = torch.cat((torch.arange(0, kept), torch.arange(lo, ctx)))
        pages = block_tables[b, keys // page_size].long()
        k = kcache[pages, :, keys % page_size, :].float().repeat_interleave(groups, dim=1).permute(1, 0, 2)
        v = vcache[pages, :, keys % page_size, :].float().repeat_interleave(groups, dim=1).permute(1, 0, 2)
        qq = q[q0:q1, : num_heads * head_dim].float().view(qlen, num_heads, head_dim).permute(1, 0, 2)
        scores = torch.matmul(qq, k.transpose(-1, -2)) * scale  # [H, qlen, T]
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        qpos = torch.arange(st[b], ctx)[:, None]
        hidden = torch.zeros(qlen, keys.numel(), dtype=torch.bool)
        if window:
            hidden = hidden | (keys[None, :] <= qpos - window)
        if chunk:
            hidden = hidden | (keys[None, :] // chunk != qpos // chunk)
        if keep_first:
            hidden = hidden & (keys[None, :] >= keep_first)
        hidden = hidden | (keys[None, :] > qpos)
        scores = scores.masked_fill(hidden, float("-inf"))
        mx = scores.max(-1, keepdim=True).values
        e = torch.exp(scores - mx)
        den = e.sum(-1, keepdim=True)
        if sinks is not None:
            den = den + torch.exp(sinks.float()[:, None, None] - mx)
        o = torch.matmul(e / den, v).permute(1, 0, 2)  # [qlen, H, DV]
        if out_table is not None:
            cs = out_table[positions[q0:q1].long()][:, None].clone()
            cs[..., 1] = -cs[..., 1]  # back by the same angle
            o = _rotate_pairs(o, cs, dv, out_pairing)
        if gate is not None:
            o = o * torch.sigmoid(gate[q0:q1, :num_heads].float())[:, :, None]
        out[q0:q1] = o.reshape(qlen, num_heads * dv).to(out.dtype)


def norm_mean2(a, b, gain_a, gain_b, eps, out):
    x, y = a.float(), b.float()
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain_a.float()
    y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * gain_b.float()
    out.copy_((0.5 * (x + y)).to(out.dtype))


def _memory_act(z, act):
    return z * torch.sigmoid(z) if act == "silu" else z


def matrix_recurrence(q, k, v, num_heads, dim, vdim, state, slots, cu_q, num_rows, out, act="none", q_scale=1.0,
                      decay_head=None, a=None, b=None, denom_floor=None, denom=None, denom_eps=0.0, qk_heads=None):
    n, H, D, V = q.shape[0], num_heads, dim, vdim
    G = qk_heads or H
    qq = (_memory_act(q[:, :G * D].float(), act).view(n, G, D) * q_scale).repeat_interleave(H // G, dim=1)
    kk = _memory_act(k[:, :G * D].float(), act).view(n, G, D).repeat_interleave(H // G, dim=1)
    vv = _memory_act(v[:, :H * V].float(), act).view(n, H, V)
    cu = cu_q.tolist()
    for r in range(num_rows):
        slot = int(slots[r])
        S = state[slot, :, :D * V].reshape(H, D, V).clone()
        nrm = state[slot, :, D * V:D * V + D].clone() if denom is not None else None
        for t in range(cu[r], cu[r + 1]):
            at = decay_head if decay_head is not None else a[t]
            bt = b[t] if b is not None else torch.ones(H)
            S = at[:, None, None] * S + bt[:, None, None] * kk[t][:, :, None] * vv[t][:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, qq[t]).reshape(-1)
            if denom is not None:
                nrm = at[:, None] * nrm + bt[:, None] * kk[t]
                denom[t] = torch.maximum((nrm * qq[t]).sum(-1).abs(), denom_floor[t]) + denom_eps
        state[slot, :, :D * V] = S.reshape(H, D * V)
        if denom is not None:
            state[slot, :, D * V:D * V + D] = nrm


def mlstm_gates(pre, bias_i, bias_f, cap, state, m_offset, slots, cu_q, num_rows, a, b, floor):
    H = pre.shape[1] // 2
    ig = cap * torch.tanh((pre[:, :H] + bias_i.float()) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((pre[:, H:] + bias_f.float()) / cap))
    cu = cu_q.tolist()
    for r in range(num_rows):
        slot = int(slots[r])
        m = state[slot, :, m_offset].clone()
        for t in range(cu[r], cu[r + 1]):
            new = torch.maximum(fg[t] + m, ig[t])
            a[t] = torch.exp(fg[t] + m - new)
            b[t] = torch.exp(ig[t] - new)
            floor[t] = torch.exp(-new)
            m = new
        state[slot, :, m_offset] = m


def group_norm_gate(o, groups, eps, weight, gate, out, denom=None):
    n, c = o.shape
    x = o.view(n, groups, c // groups)
    if denom is not None:
        x = x / denom[:, :, None]
    x = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, c) * weight.float()
    if gate is not None:
        x = x * torch.sigmoid(gate[:, :c].float())
    out.copy_(x.to(out.dtype))


def rglru_scan(u, pre, bias_r, bias_i, lam, y, y_act, cmul, state, slots, cu_q, num_rows, out, blocks):
    n, c = u.shape
    bw = c // blocks
    gates = pre.reshape(2, blocks, n, bw).permute(0, 2, 1, 3).reshape(2, n, c)
    r = torch.sigmoid(gates[0] + bias_r.float().reshape(-1))
    i = torch.sigmoid(gates[1] + bias_i.float().reshape(-1))
    log_a = -cmul * r * torch.nn.functional.softplus(lam.float())
    a = torch.exp(log_a)
    x = torch.sqrt(-torch.expm1(2 * log_a)) * i * u.float()
    yy = y[:, :c].float()
    if y_act:
        yy = 0.5 * yy * (1 + torch.tanh(math.sqrt(2 / math.pi) * (yy + 0.044715 * yy ** 3)))
    cu = cu_q.tolist()
    for row in range(num_rows):
        slot = int(slots[row])
        S = state[slot].clone()
        for t in range(cu[row], cu[row + 1]):
            S = a[t] * S + x[t]
            out[t] = (S * yy[t]).to(out.dtype)
        state[slot] = S


def add_scaled_norm2(deltas, residual, gain1, gain2, gain_offset, eps, out1, out2):
    for d, sc in deltas:
        residual += sc * d.float()
    x = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps)
    if out1 is not None:
        out1.copy_((x * (gain1.float() + gain_offset)).to(out1.dtype))
    if out2 is not None:
        out2.copy_((x * (gain2.float() + gain_offset)).to(out2.dtype))


def stream_norm(residual, gain, gain_offset, eps):
    residual.copy_(residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps) * (gain.float() + gain_offset))


def softcap(x, cap):
    x.copy_(cap * torch.tanh(x / cap))


def delta_recurrence(q, k, v, beta, g_raw, g_bias, a_log, num_heads, qk_heads, dim, vdim, state, slots, cu_q,
                     num_rows, out, act="silu", unit_eps=1e-6, q_scale=1.0, work=None):
    n, H, G, D, V = q.shape[0], num_heads, qk_heads, dim, vdim
    qq = _memory_act(q[:, :G * D].float(), act).view(n, G, D)
    kk = _memory_act(k[:, :G * D].float(), act).view(n, G, D)
    if unit_eps is not None:
        qq = qq * torch.rsqrt(qq.pow(2).sum(-1, keepdim=True) + unit_eps)
        kk = kk * torch.rsqrt(kk.pow(2).sum(-1, keepdim=True) + unit_eps)
    qq = (qq * q_scale).repeat_interleave(H // G, dim=1)
    kk = kk.repeat_interleave(H // G, dim=1)
    vv = _memory_act(v[:, :H * V].float(), act).view(n, H, V)
    bb = torch.sigmoid(beta[:, :H].float())
    gg = torch.exp(-torch.exp(a_log.float())[None, :, None]
                   * torch.nn.functional.softplus(g_raw + g_bias.float().reshape(-1)).view(n, H, D))
    cu = cu_q.tolist()
    for r in range(num_rows):
        slot = int(slots[r])
        S = state[slot].reshape(H, D, V).clone()
        for t in range(cu[r], cu[r + 1]):
            S = gg[t][:, :, None] * S
            u = bb[t][:, None] * (vv[t] - torch.einsum("hdv,hd->hv", S, kk[t]))
            S = S + kk[t][:, :, None] * u[:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, qq[t]).reshape(-1)
        state[slot] = S.reshape(H, D * V)


def ssm_gates(x, bias, a_log, a, b):
    dt = torch.nn.functional.softplus(x.float() + bias.float())
    a.copy_(torch.exp(-torch.exp(a_log.float()) * dt))
    b.copy_(dt)


def gate_group_norm(o, groups, eps, weight, out, z=None, skip=None, x=None, x_act="none", head_width=None):
    n, c = o.shape
    y = o
    if skip is not None:
        y = y + skip.float().repeat_interleave(head_width or c) * _memory_act(x[:, :c].float(), x_act)
    if z is not None:
        zz = z[:, :c].float()
        y = y * zz * torch.sigmoid(zz)
    y = y.view(n, groups, c // groups)
    y = (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, c) * weight.float()
    out.copy_(y.to(out.dtype))


ALL = ["gemm_smallm", "gemm_smallm_gated", "check_status", "embedding", "add_rmsnorm", "silu_mul", "rope_table", "rope_kv_write",
       "attention_scratch_bytes", "paged_attention", "argmax", "repetition_penalty", "sample",
       "stream_inject", "add_norm_grouped", "glu_act", "causal_taps", "latent_prep", "rope_inplace",
       "latent_attention_scratch_bytes", "latent_attention", "heads_gate", "moe_tile_rows", "moe_max_tiles",
       "moe_route", "moe_up", "moe_down", "moe_combine", "unary_act", "qk_prep", "paged_attention_masked",
       "norm_mean2", "matrix_recurrence", "mlstm_gates", "group_norm_gate", "rglru_scan", "add_cast", "token_gate",
       "depth_mix", "add_scaled_norm2", "stream_norm", "softcap", "delta_recurrence", "ssm_gates", "gate_group_norm"]


def install(monkeypatch) -> None:
    """Replace the CUDA kernels of the package by these restatements (host-logic tests)."""
    import sys

    import emberserve_b200.kernels as K

    me = sys.modules[__name__]
    for name in ALL:
        monkeypatch.setattr(K, name, getattr(me, name))
