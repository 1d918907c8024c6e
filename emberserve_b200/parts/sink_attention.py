"""Grouped-query attention over a paged cache with the options that newer decoders combine:

* the values may be the keys themselves as projected, before rotation and norm (no value projection);
* q and k, after a rotation of the first `rotary_dim` numbers of each head, may be divided by
  their root mean square per head (a norm without gain);
* a chunk mask: the query at position p sees key j <= p only if ``j // chunk == p // chunk``,
  chunks counted from position 0 of the request, wherever a prompt was cut; and / or a window;
* a sink: ``exp(sink[h])`` joins the softmax denominator of head h; it has no key and no value;
* a gate per (token, head): head h's output is multiplied by ``sigmoid(x Wg^T)[h]``;
* first keys that stay visible: with `keep_first`, keys at positions below it are seen by every later
  query beside the window (or chunk), at their true positions; the cache holds their pages to the end;
* value heads of a size of their own (`v_head_dim`), divided by their root mean square (`v_norm_eps`, no
  gain) and turned by their position over their whole length (`value_position`, a rotary spec over
  `v_head_dim` numbers) before they are cached; each head's sum over the values is then turned back by
  the query's position, so that the output depends on distances only.

* a short causal convolution over time on every channel of q, k and v right behind the projections
  (`conv_taps`; the last taps - 1 projected rows of a request are state of the mixer);
* gains on the normed q and k (`q_norm_name`, `k_norm_name`: [head_dim], shared by the heads), and the
  norm BEFORE the rotation instead of behind it (`norm_before_rotation`);
* capped scores: a scaled score s enters the softmax as ``softcap * tanh(s / softcap)``;
* a bias on the output projection.

``[q | k | (v) | gate] = x W^T + b`` is one product; one kernel rotates, norms and writes the
cache; the attention kernel applies mask, sink and gate; then ``o = attn Wo^T``.  Scores, softmax,
rotation and the unit norms are 32-bit.  With a chunk mask the cache gives back the pages of
chunks that are over (``PagedKV.chunk``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.attention import decode_splits
from emberserve_b200.parts.base import (Mixer, PagedKV, PagedKVHandle, ParamSpec, Part, Source, StepContext,
                                        build_part, register_part)
from emberserve_b200.parts.conv import CausalTapsSpec
from emberserve_b200.parts.linear import linear


@dataclass(frozen=True)
class SinkAttentionSpec:
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    position: Any  # spec of a rotary position encoding, or None
    # checkpoint tensors (full names); a bias name may be None
    q_name: str
    k_name: str
    o_name: str
    v_name: str | None = None  # None: the values are the keys as projected
    q_bias_name: str | None = None
    k_bias_name: str | None = None
    v_bias_name: str | None = None
    sink_name: str | None = None  # [num_heads]
    gate_name: str | None = None  # [num_heads, hidden]
    qk_norm_eps: float | None = None  # unit RMS of q and k per head after the rotation
    chunk: int | None = None
    window: int | None = None
    kind: str = "sink_attention"
    keep_first: int = 0  # keys below this position stay visible beside the window / chunk
    v_head_dim: int | None = None  # numbers per value head (None: head_dim)
    v_norm_eps: float | None = None  # unit RMS of every value head
    value_position: Any = None  # rotary spec over v_head_dim numbers: values turned when cached, the sum turned back
    conv_taps: int = 1  # > 1: a causal convolution of that many taps on q, k and v
    q_conv_name: str | None = None  # checkpoint tensors [channels, taps]
    k_conv_name: str | None = None
    v_conv_name: str | None = None
    q_norm_name: str | None = None  # [head_dim] gains of the normed q and k (with qk_norm_eps)
    k_norm_name: str | None = None
    norm_before_rotation: bool = False
    softcap: float | None = None
    o_bias_name: str | None = None


@register_part("mixer", "sink_attention")
class SinkAttention(Mixer):
    wqkv: torch.Tensor
    wo: torch.Tensor
    bqkv: torch.Tensor | None = None
    sink: torch.Tensor | None = None
    bo: torch.Tensor | None = None
    q_gain: torch.Tensor | None = None
    k_gain: torch.Tensor | None = None

    def __init__(self, spec: SinkAttentionSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim % 8 or spec.head_dim > 256:
            raise ValueError(f"head_dim={spec.head_dim}: the attention kernels take multiples of 8 up to 256")
        self.v_dim = spec.head_dim if spec.v_head_dim is None else spec.v_head_dim
        if self.v_dim % 8 or self.v_dim > 256:
            raise ValueError(f"v_head_dim={self.v_dim}: the attention kernels take multiples of 8 up to 256")
        if spec.v_name is None and (self.v_dim != spec.head_dim or spec.v_norm_eps is not None
                                    or spec.value_position is not None):
            raise ValueError("values that are the keys as projected have the keys' size, no norm and no rotation")
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * spec.head_dim
        self.o_size = spec.num_heads * self.v_dim
        self.v_cols = 0 if spec.v_name is None else spec.num_kv_heads * self.v_dim
        self.gate_at = self.q_size + self.kv_size + self.v_cols
        # the gate's columns are padded so that a row of the product stays 16-byte aligned
        self.gate_cols = 0 if spec.gate_name is None else -(-spec.num_heads // 8) * 8
        self.cols = self.gate_at + self.gate_cols
        self.position = self.shared.get("position", spec.position) if spec.position is not None else None
        self.value_position = (self.shared.get("position", spec.value_position)
                               if spec.value_position is not None else None)
        if self.value_position is not None and self.value_position.spec.rotary_dim != self.v_dim:
            raise ValueError("the rotation of the values covers the whole value head")
        self._sink32: torch.Tensor | None = None
        if (spec.q_norm_name is None) != (spec.k_norm_name is None) or (
                spec.q_norm_name is not None and spec.qk_norm_eps is None):
            raise ValueError("gains on q and k come in pairs and need qk_norm_eps")
        self.conv = None
        if spec.conv_taps > 1 or spec.q_conv_name is not None:
            if spec.v_name is None or None in (spec.q_conv_name, spec.k_conv_name, spec.v_conv_name):
                raise ValueError("the convolution filters projected q, k and v and needs a weight for each")
            q, kv = self.q_size, self.kv_size
            self.conv = build_part("conv", CausalTapsSpec(
                self.gate_at, spec.conv_taps, spec.q_conv_name, identity=False,
                weight_parts=((spec.q_conv_name, 0, q), (spec.k_conv_name, q, q + kv),
                              (spec.v_conv_name, q + kv, self.gate_at))), prefix + ".conv", self.shared)
        self._conv_state = self.conv.cache_need() if self.conv is not None else None

    def children(self) -> dict[str, Part]:
        return {} if self.conv is None else {"conv": self.conv}

    def cache_need(self):
        s: SinkAttentionSpec = self.spec
        pages = PagedKV(s.num_kv_heads, s.head_dim, s.window, s.chunk, keep_first=int(s.keep_first or 0),
                        v_head_dim=None if self.v_dim == s.head_dim else self.v_dim)
        return pages if self._conv_state is None else (pages, self._conv_state)

    def param_specs(self) -> dict[str, ParamSpec]:
        s: SinkAttentionSpec = self.spec
        q, kv = self.q_size, self.kv_size
        rows = [(s.q_name, s.q_bias_name, (0, q)), (s.k_name, s.k_bias_name, (q, q + kv))]
        if s.v_name is not None:
            rows.append((s.v_name, s.v_bias_name, (q + kv, q + kv + self.v_cols)))
        if s.gate_name is not None:
            rows.append((s.gate_name, None, (self.gate_at, self.gate_at + s.num_heads)))
        # (rows that no tensor fills, the gate's padding and absent biases, stay zero)
        specs = {
            "wqkv": ParamSpec((self.cols, s.hidden), [Source(n, r) for n, _, r in rows]),
            "wo": ParamSpec((s.hidden, self.o_size), [Source(s.o_name)]),
        }
        biased = [(b, r) for _, b, r in rows if b is not None]
        if biased:
            specs["bqkv"] = ParamSpec((self.cols,), [Source(b, r) for b, r in biased], init="bias")
        if s.sink_name is not None:
            specs["sink"] = ParamSpec((s.num_heads,), [Source(s.sink_name)], init="bias")
        if s.o_bias_name is not None:
            specs["bo"] = ParamSpec((s.hidden,), [Source(s.o_bias_name)], init="bias")
        if s.q_norm_name is not None:
            specs["q_gain"] = ParamSpec((s.head_dim,), [Source(s.q_norm_name)], init="ones")
            specs["k_gain"] = ParamSpec((s.head_dim,), [Source(s.k_norm_name)], init="ones")
        return specs

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        super().bind(params)
        self._sink32 = None if self.sink is None else self.sink.float().contiguous()

    def streamed_params(self) -> list[str]:
        return ["wqkv", "wo"]

    def scratch_elements_per_token(self) -> int:
        return self.cols + self.o_size + self.spec.hidden  # (a convolution's output is its own part's)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        s: SinkAttentionSpec = self.spec
        n, b = ctx.num_tokens, ctx.num_rows
        conv_cache = None
        if self._conv_state is not None:
            cache, conv_cache = cache
        proj = ctx.scratch("sink_qkv", (n, self.cols), ctx.dtype)
        linear(x, self.wqkv, self.bqkv, proj, ctx.scratch)
        gate = proj[:, self.gate_at:self.gate_at + self.gate_cols] if self.gate_cols else None
        if self.conv is not None:  # (the gate's columns, if any, stay where they are)
            proj = self.conv.forward(proj[:, :self.gate_at], ctx, conv_cache)
        table, rot, pairing = None, 0, "half"
        if self.position is not None:
            r = self.position.rotary(ctx.device)
            if r is not None:
                (table, rot), pairing = r, self.position.pairing
        vtable, vpairing = None, "half"
        if self.value_position is not None:
            vtable, vpairing = self.value_position.rotary(ctx.device)[0], self.value_position.pairing
        K.qk_prep(proj, s.num_heads, s.num_kv_heads, s.head_dim, ctx.positions, ctx.row_of_token, table, rot,
                  pairing, s.qk_norm_eps, cache.k, cache.v, cache.block_tables, s.v_name is None, cache.write,
                  v_norm_eps=s.v_norm_eps, v_table=vtable, v_pairing=vpairing, q_gain=self.q_gain,
                  k_gain=self.k_gain, norm_first=s.norm_before_rotation)
        out = ctx.scratch("attn_out", (n, self.o_size), ctx.dtype)
        extras = dict(keep_first=int(s.keep_first or 0), out_table=vtable, out_pairing=vpairing,
                      positions=ctx.positions if vtable is not None else None, softcap=s.softcap)
        kern = ctx.extra.get("attn_kernel", "auto")
        if ctx.all_decode and n == b:
            # one token per row: the keys of a row are split over blocks when rows are few.  A chunk
            # or a window bounds the keys a query reads, whatever the context.
            reach = min(x for x in (ctx.max_ctx_len, s.chunk, s.window) if x)
            if s.keep_first and reach < ctx.max_ctx_len:
                reach = min(ctx.max_ctx_len, reach + int(s.keep_first))
            splits = decode_splits(b, s.num_kv_heads, reach, K.sm_count(ctx.device))
            scratch = None
            if splits > 1:
                nbytes = K.attention_scratch_bytes(b, s.num_heads, self.v_dim, splits)
                scratch = ctx.scratch("attn_partials", (nbytes // 4,), torch.float32)
            K.paged_attention_masked(proj, out, cache.k, cache.v, cache.block_tables, ctx.cu_q, ctx.starts, b, n,
                                     s.num_heads, s.num_kv_heads, s.head_dim, s.scale, 1, window=s.window,
                                     chunk=s.chunk, sinks=self._sink32, gate=gate, splits=splits, scratch=scratch,
                                     kernel=kern, **extras)
        else:
            K.paged_attention_masked(proj, out, cache.k, cache.v, cache.block_tables, ctx.cu_q, ctx.starts, b, n,
                                     s.num_heads, s.num_kv_heads, s.head_dim, s.scale, ctx.max_q_len,
                                     window=s.window, chunk=s.chunk, sinks=self._sink32, gate=gate, kernel=kern,
                                     **extras)
        y = ctx.scratch("mixer_out", (n, s.hidden), ctx.dtype)
        return linear(out, self.wo, self.bo, y, ctx.scratch)
