"""Mixers that keep state of fixed size per request (``FixedState``) instead of a growing cache.

* ``decay_linear_attention``: linear attention with a fixed decay per head ("lightning attention"):
  ``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with q, k, v passed through an
  activation; all heads together are RMS-normed with a gain, gated by ``sigmoid(x Wg^T)`` and
  projected.
* ``mlstm``: the matrix memory of the xLSTM with exponential gating: per head a log input gate
  ``i = cap tanh(x_i / cap)`` and a log forget gate ``f = logsigmoid(cap tanh(x_f / cap))``, a
  running maximum ``m_t = max(f + m_(t-1), i)`` that starts at 0, ``S_t = exp(f + m_(t-1) - m_t)
  S_(t-1) + exp(i - m_t) k v^T``, the same for a normaliser n with k alone, ``o = S_t^T q /
  (max(|n_t . q|, exp(-m_t)) + denom_eps)``; each head's o is brought to unit RMS, then gain, gate
  and projection.
* ``rglru``: two branches, ``y = gelu_tanh(x Wy^T + by)`` and ``u = conv(x Wx^T + bx)`` (a short
  causal convolution per channel); per channel ``r = sigmoid(Ra u + bra)``, ``i = sigmoid(Ri u +
  bri)`` with block-diagonal Ra, Ri; ``a = exp(-c r softplus(lam))``, ``S_t = a S_(t-1) + sqrt(1 -
  a^2) i u``; the output is ``(S * y) Wo^T``.

States, gates, decays and every product with a state are 32-bit; the projections and the
convolution are in the activation type.  Gate pre-activations are products with 32-bit results.
* ``selective_state_space``: a state space with a scalar decay and step size per head and token, B and C
  shared by groups of heads, a skip, a gate before a grouped norm (see the class).
* ``channel_delta``: the delta rule with a decay per head and key channel (see the class).

The same kernels walk a request's tokens in order in prompts, portions and single tokens.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (FixedState, FixedStateHandle, Mixer, ParamSpec, Part, Source, StepContext,
                                        build_part, register_part)
from emberserve_b200.parts.conv import CausalTapsSpec
from emberserve_b200.parts.linear import bmm_f32_out, linear, linear_f32_out


@dataclass(frozen=True)
class DecayLinearAttentionSpec:
    hidden: int
    num_heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]  # one per head
    eps: float
    # checkpoint tensors (full names)
    q_name: str
    k_name: str
    v_name: str
    g_name: str
    o_name: str
    norm_name: str
    activation: str = "silu"  # on q, k and v: one of kernels.MEMORY_INPUT_ACTIVATIONS
    norm_groups: int = 1  # 1: all heads are normed together
    kind: str = "decay_linear_attention"


@register_part("mixer", "decay_linear_attention")
class DecayLinearAttention(Mixer):
    wqkvg: torch.Tensor
    wo: torch.Tensor
    norm: torch.Tensor

    def __init__(self, spec: DecayLinearAttentionSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if len(spec.decay) != spec.num_heads:
            raise ValueError(f"{spec.num_heads} heads need as many decays, got {len(spec.decay)}")
        if spec.dim > 256:
            raise ValueError(f"dim={spec.dim}: the memory kernel holds at most 256 rows per head")
        self.qk, self.vv = spec.num_heads * spec.dim, spec.num_heads * spec.vdim
        self._decay: torch.Tensor | None = None

    def cache_need(self) -> FixedState:
        s: DecayLinearAttentionSpec = self.spec
        return FixedState((s.num_heads, s.dim * s.vdim), "float32")

    def param_specs(self) -> dict[str, ParamSpec]:
        s: DecayLinearAttentionSpec = self.spec
        qk, vv = self.qk, self.vv
        return {
            "wqkvg": ParamSpec((2 * qk + 2 * vv, s.hidden), [
                Source(s.q_name, (0, qk)), Source(s.k_name, (qk, 2 * qk)), Source(s.v_name, (2 * qk, 2 * qk + vv)),
                Source(s.g_name, (2 * qk + vv, 2 * qk + 2 * vv))]),
            "wo": ParamSpec((s.hidden, vv), [Source(s.o_name)]),
            "norm": ParamSpec((vv,), [Source(s.norm_name)], init="ones"),
        }

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        super().bind(params)
        self._decay = torch.tensor(self.spec.decay, dtype=torch.float32, device=self.wo.device)

    def streamed_params(self) -> list[str]:
        return ["wqkvg", "wo"]

    def scratch_elements_per_token(self) -> int:
        return 2 * self.qk + 2 * self.vv + 3 * self.vv + self.spec.hidden  # (the 32-bit read counts twice)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: FixedStateHandle) -> torch.Tensor:
        s: DecayLinearAttentionSpec = self.spec
        n, qk, vv = ctx.num_tokens, self.qk, self.vv
        proj = ctx.scratch("memory_qkvg", (n, 2 * qk + 2 * vv), ctx.dtype)
        linear(x, self.wqkvg, None, proj, ctx.scratch)
        read = ctx.scratch("memory_read", (n, vv), torch.float32)
        K.matrix_recurrence(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vv], s.num_heads, s.dim,
                            s.vdim, cache.state, cache.slots, ctx.cu_q, ctx.num_rows, read, act=s.activation,
                            decay_head=self._decay)
        gated = ctx.scratch("memory_gated", (n, vv), ctx.dtype)
        K.group_norm_gate(read, s.norm_groups, s.eps, self.norm, proj[:, 2 * qk + vv:], gated)
        y = ctx.scratch("memory_out", (n, s.hidden), ctx.dtype)
        return linear(gated, self.wo, None, y, ctx.scratch)


@dataclass(frozen=True)
class MLSTMSpec:
    hidden: int
    num_heads: int
    dim: int
    vdim: int
    gate_cap: float
    eps: float
    # checkpoint tensors (full names)
    q_name: str
    k_name: str
    v_name: str
    g_name: str
    o_name: str
    norm_name: str
    i_name: str
    i_bias_name: str
    f_name: str
    f_bias_name: str
    denom_eps: float = 1e-6
    kind: str = "mlstm"


@register_part("mixer", "mlstm")
class MLSTM(Mixer):
    wqkvg: torch.Tensor
    wif: torch.Tensor
    bi: torch.Tensor
    bf: torch.Tensor
    wo: torch.Tensor
    norm: torch.Tensor

    def __init__(self, spec: MLSTMSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.dim > 256:
            raise ValueError(f"dim={spec.dim}: the memory kernel holds at most 256 rows per head")
        self.qk, self.vv = spec.num_heads * spec.dim, spec.num_heads * spec.vdim
        self.per_head = spec.dim * spec.vdim + spec.dim + 1  # S, the normaliser, the running maximum

    def cache_need(self) -> FixedState:
        return FixedState((self.spec.num_heads, self.per_head), "float32")

    def param_specs(self) -> dict[str, ParamSpec]:
        s: MLSTMSpec = self.spec
        qk, vv, h = self.qk, self.vv, s.num_heads
        return {
            "wqkvg": ParamSpec((2 * qk + 2 * vv, s.hidden), [
                Source(s.q_name, (0, qk)), Source(s.k_name, (qk, 2 * qk)), Source(s.v_name, (2 * qk, 2 * qk + vv)),
                Source(s.g_name, (2 * qk + vv, 2 * qk + 2 * vv))]),
            "wif": ParamSpec((2 * h, s.hidden), [Source(s.i_name, (0, h)), Source(s.f_name, (h, 2 * h))]),
            "bi": ParamSpec((h,), [Source(s.i_bias_name)], init="bias"),
            "bf": ParamSpec((h,), [Source(s.f_bias_name)], init="bias"),
            "wo": ParamSpec((s.hidden, vv), [Source(s.o_name)]),
            "norm": ParamSpec((vv,), [Source(s.norm_name)], init="ones"),
        }

    def streamed_params(self) -> list[str]:
        return ["wqkvg", "wo"]

    def scratch_elements_per_token(self) -> int:
        return 2 * self.qk + 2 * self.vv + 3 * self.vv + self.spec.hidden + 12 * self.spec.num_heads

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: FixedStateHandle) -> torch.Tensor:
        s: MLSTMSpec = self.spec
        n, qk, vv, h = ctx.num_tokens, self.qk, self.vv, s.num_heads
        proj = ctx.scratch("memory_qkvg", (n, 2 * qk + 2 * vv), ctx.dtype)
        linear(x, self.wqkvg, None, proj, ctx.scratch)
        pre = ctx.scratch("mlstm_pre", (n, 2 * h), torch.float32)
        linear_f32_out(x, self.wif, pre)
        gates = ctx.scratch("mlstm_gates", (4, n, h), torch.float32)  # decay, input scale, floor, denominator
        K.mlstm_gates(pre, self.bi, self.bf, s.gate_cap, cache.state, self.per_head - 1, cache.slots, ctx.cu_q,
                      ctx.num_rows, gates[0], gates[1], gates[2])
        read = ctx.scratch("memory_read", (n, vv), torch.float32)
        K.matrix_recurrence(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + vv], h, s.dim, s.vdim,
                            cache.state, cache.slots, ctx.cu_q, ctx.num_rows, read, q_scale=s.dim ** -0.5,
                            a=gates[0], b=gates[1], denom_floor=gates[2], denom=gates[3], denom_eps=s.denom_eps)
        gated = ctx.scratch("memory_gated", (n, vv), ctx.dtype)
        K.group_norm_gate(read, h, s.eps, self.norm, proj[:, 2 * qk + vv:], gated, denom=gates[3])
        y = ctx.scratch("memory_out", (n, s.hidden), ctx.dtype)
        return linear(gated, self.wo, None, y, ctx.scratch)


@dataclass(frozen=True)
class RGLRUSpec:
    hidden: int
    width: int  # channels of both branches
    blocks: int  # of the block-diagonal gate matrices
    taps: int  # of the convolution; 1 keeps no state
    # checkpoint tensors (full names)
    y_name: str
    y_bias_name: str
    x_name: str
    x_bias_name: str
    conv_name: str
    conv_bias_name: str
    ra_name: str  # [blocks, width / blocks, width / blocks], [out, in] per block
    ra_bias_name: str
    ri_name: str
    ri_bias_name: str
    lam_name: str
    o_name: str
    decay_scale: float = 8.0  # c in a = exp(-c r softplus(lam))
    kind: str = "rglru"


@register_part("mixer", "rglru")
class RGLRU(Mixer):
    wyx: torch.Tensor
    byx: torch.Tensor
    wra: torch.Tensor
    wri: torch.Tensor
    bra: torch.Tensor
    bri: torch.Tensor
    lam: torch.Tensor
    wo: torch.Tensor

    def __init__(self, spec: RGLRUSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.blocks <= 0 or spec.width % spec.blocks:
            raise ValueError(f"{spec.width} channels do not split into {spec.blocks} equal blocks")
        self.conv = build_part("conv", CausalTapsSpec(spec.width, spec.taps, spec.conv_name, identity=False,
                                                      bias_name=spec.conv_bias_name), prefix + ".conv", self.shared)
        self._conv_state = self.conv.cache_need()

    def children(self) -> dict[str, Part]:
        return {"conv": self.conv}

    def cache_need(self):
        state = FixedState((self.spec.width,), "float32")
        return state if self._conv_state is None else (self._conv_state, state)

    def param_specs(self) -> dict[str, ParamSpec]:
        s: RGLRUSpec = self.spec
        c, b = s.width, s.blocks
        bw = c // b
        return {
            "wyx": ParamSpec((2 * c, s.hidden), [Source(s.y_name, (0, c)), Source(s.x_name, (c, 2 * c))]),
            "byx": ParamSpec((2 * c,), [Source(s.y_bias_name, (0, c)), Source(s.x_bias_name, (c, 2 * c))], init="bias"),
            "wra": ParamSpec((b, bw, bw), [Source(s.ra_name)]),
            "wri": ParamSpec((b, bw, bw), [Source(s.ri_name)]),
            "bra": ParamSpec((b, bw), [Source(s.ra_bias_name)], init="bias"),
            "bri": ParamSpec((b, bw), [Source(s.ri_bias_name)], init="bias"),
            "lam": ParamSpec((c,), [Source(s.lam_name)], init="bias"),
            "wo": ParamSpec((s.hidden, c), [Source(s.o_name)]),
        }

    def streamed_params(self) -> list[str]:
        return ["wyx", "wo"]

    def scratch_elements_per_token(self) -> int:
        return 2 * self.spec.width + 4 * self.spec.width + self.spec.width + self.spec.hidden

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        s: RGLRUSpec = self.spec
        n, c, b = ctx.num_tokens, s.width, s.blocks
        bw = c // b
        conv_cache, state = (None, cache) if self._conv_state is None else cache
        yx = ctx.scratch("rglru_yx", (n, 2 * c), ctx.dtype)
        linear(x, self.wyx, self.byx, yx, ctx.scratch)
        u = self.conv.forward(yx[:, c:], ctx, conv_cache)
        pre = ctx.scratch("rglru_pre", (2, b, n, bw), torch.float32)
        ub = u.view(n, b, bw).transpose(0, 1)
        bmm_f32_out(ub, self.wra.transpose(1, 2), pre[0])
        bmm_f32_out(ub, self.wri.transpose(1, 2), pre[1])
        out = ctx.scratch("rglru_out", (n, c), ctx.dtype)
        K.rglru_scan(u, pre, self.bra, self.bri, self.lam, yx[:, :c], True, s.decay_scale, state.state,
                     state.slots, ctx.cu_q, ctx.num_rows, out, b)
        y = ctx.scratch("memory_out", (n, s.hidden), ctx.dtype)
        return linear(out, self.wo, None, y, ctx.scratch)


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


@dataclass(frozen=True)
class SelectiveStateSpaceSpec:
    hidden: int
    num_heads: int
    vdim: int  # channels per head
    state: int  # N: rows of a head's state
    groups: int  # heads that share one B and C: head h reads group h // (num_heads / groups)
    norm_groups: int
    taps: int  # of the convolution over x, B and C; 1 keeps no state
    eps: float
    # checkpoint tensors (full names)
    in_name: str  # [2 inner + 2 groups N + heads, hidden]: z | x | B | C | dt
    conv_name: str  # [inner + 2 groups N, taps]
    conv_bias_name: str
    dt_bias_name: str  # [heads]
    a_log_name: str  # [heads]
    d_name: str  # [heads]
    norm_name: str  # [inner]
    o_name: str  # [hidden, inner]
    kind: str = "selective_state_space"


@register_part("mixer", "selective_state_space")
class SelectiveStateSpace(Mixer):
    """A selective state space with a scalar decay per head (the "state-space duality" form):

        [z | x | B | C | dt] = h Win^T;   (x, B, C) <- silu(conv(x, B, C));   dt <- softplus(dt + dt_bias)
        S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,       y_t = S_t^T C_t + D x_t        per head
        out = (rms_groups(y * silu(z)) * norm) Wo^T

    The recurrence is the matrix memory of ``ems_matrix_recurrence`` with k = B, q = C, v = x, a per-token
    decay and input scale, and B / C heads shared by groups of heads.  dt, the decay, the state and the
    gated norm are 32-bit."""

    win: torch.Tensor
    dt_bias: torch.Tensor
    a_log: torch.Tensor
    skip: torch.Tensor
    norm: torch.Tensor
    wo: torch.Tensor

    def __init__(self, spec: SelectiveStateSpaceSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.groups <= 0 or spec.num_heads % spec.groups:
            raise ValueError(f"{spec.num_heads} heads do not split into {spec.groups} groups")
        if spec.state > 256:
            raise ValueError(f"state={spec.state}: the memory kernel holds at most 256 rows per head")
        self.inner = spec.num_heads * spec.vdim
        if spec.norm_groups <= 0 or self.inner % spec.norm_groups:
            raise ValueError(f"{self.inner} channels do not split into {spec.norm_groups} norm groups")
        self.gn = spec.groups * spec.state
        self.conv_width = self.inner + 2 * self.gn
        self.dt_at = 2 * self.inner + 2 * self.gn
        self.rows = self.dt_at + spec.num_heads
        self.conv = build_part("conv", CausalTapsSpec(self.conv_width, spec.taps, spec.conv_name, identity=False,
                                                      bias_name=spec.conv_bias_name), prefix + ".conv", self.shared)
        self._conv_state = self.conv.cache_need()

    def children(self) -> dict[str, Part]:
        return {"conv": self.conv}

    def cache_need(self):
        s: SelectiveStateSpaceSpec = self.spec
        state = FixedState((s.num_heads, s.state * s.vdim), "float32")
        return state if self._conv_state is None else (self._conv_state, state)

    def param_specs(self) -> dict[str, ParamSpec]:
        s: SelectiveStateSpaceSpec = self.spec
        h = s.num_heads
        return {
            # (rows past the tensor's, padding to a multiple of 8, stay zero)
            "win": ParamSpec((_pad8(self.rows), s.hidden), [Source(s.in_name, (0, self.rows))]),
            "dt_bias": ParamSpec((h,), [Source(s.dt_bias_name)], init="bias"),
            "a_log": ParamSpec((h,), [Source(s.a_log_name)], init="bias"),
            "skip": ParamSpec((h,), [Source(s.d_name)], init="ones"),
            "norm": ParamSpec((self.inner,), [Source(s.norm_name)], init="ones"),
            "wo": ParamSpec((s.hidden, self.inner), [Source(s.o_name)]),
        }

    def streamed_params(self) -> list[str]:
        return ["win", "wo"]

    def scratch_elements_per_token(self) -> int:
        return _pad8(self.rows) + 3 * self.inner + self.spec.hidden + 4 * self.spec.num_heads

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        s: SelectiveStateSpaceSpec = self.spec
        n, inner, gn, h = ctx.num_tokens, self.inner, self.gn, s.num_heads
        conv_cache, state = (None, cache) if self._conv_state is None else cache
        proj = ctx.scratch("ssm_in", (n, _pad8(self.rows)), ctx.dtype)
        linear(x, self.win, None, proj, ctx.scratch)
        xbc = self.conv.forward(proj[:, inner:inner + self.conv_width], ctx, conv_cache)
        gates = ctx.scratch("ssm_gates", (2, n, h), torch.float32)
        K.ssm_gates(proj[:, self.dt_at:self.dt_at + h], self.dt_bias, self.a_log, gates[0], gates[1])
        read = ctx.scratch("memory_read", (n, inner), torch.float32)
        K.matrix_recurrence(xbc[:, inner + gn:], xbc[:, inner:inner + gn], xbc[:, :inner], h, s.state, s.vdim,
                            state.state, state.slots, ctx.cu_q, ctx.num_rows, read, act="silu", a=gates[0],
                            b=gates[1], qk_heads=s.groups)
        gated = ctx.scratch("memory_gated", (n, inner), ctx.dtype)
        K.gate_group_norm(read, s.norm_groups, s.eps, self.norm, gated, z=proj[:, :inner], skip=self.skip,
                          x=xbc[:, :inner], x_act="silu", head_width=s.vdim)
        y = ctx.scratch("memory_out", (n, s.hidden), ctx.dtype)
        return linear(gated, self.wo, None, y, ctx.scratch)


@dataclass(frozen=True)
class ChannelDeltaSpec:
    hidden: int
    num_heads: int  # value heads
    qk_heads: int  # heads of q and k: head h reads q / k head h // (num_heads / qk_heads)
    dim: int
    vdim: int
    taps: int  # of the convolutions on q, k and v; 1 keeps no state
    decay_rank: int  # inner size of the two-step decay projection
    gate_rank: int  # inner size of the two-step output-gate projection
    eps: float
    # checkpoint tensors (full names)
    q_name: str
    k_name: str
    v_name: str
    q_conv_name: str
    k_conv_name: str
    v_conv_name: str
    beta_name: str  # [heads, hidden]
    a_log_name: str  # [heads]
    decay_in_name: str  # [decay_rank, hidden]
    decay_out_name: str  # [heads * dim, decay_rank]
    decay_bias_name: str  # [heads * dim]
    gate_in_name: str  # [gate_rank, hidden]
    gate_out_name: str  # [heads * vdim, gate_rank]
    norm_name: str  # [vdim], shared by the heads
    o_name: str
    unit_eps: float = 1e-6  # q and k become x / sqrt(sum(x^2) + unit_eps) per head
    kind: str = "channel_delta"


@register_part("mixer", "channel_delta")
class ChannelDelta(Mixer):
    """The delta rule with a decay per head and key channel:

        q, k, v <- silu(conv(h Wq^T)), ...;   q, k <- unit vectors per head;   q <- q dim^(-1/2)
        beta = sigmoid(h Wb^T);   g = exp(-exp(A_log) softplus((h Wa1^T) Wa2^T + dt_bias))     [heads, dim]
        S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                   per head
        out = (rms(o) * norm * sigmoid((h Wg1^T) Wg2^T)) Wo^T

    One product gives ``[q | k | v | a1 | g1 | b]``; the convolution runs over the q, k and v columns;
    the second steps of the decay and of the gate are products of their own (the decay's with a 32-bit
    result); ``ems_delta_recurrence`` does the activation, the unit norms, beta, the decay and the rule
    itself in 32 bits."""

    win: torch.Tensor
    wa2: torch.Tensor
    wg2: torch.Tensor
    dt_bias: torch.Tensor
    a_log: torch.Tensor
    norm: torch.Tensor
    wo: torch.Tensor

    def __init__(self, spec: ChannelDeltaSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.qk_heads <= 0 or spec.num_heads % spec.qk_heads:
            raise ValueError(f"{spec.num_heads} heads over {spec.qk_heads} heads of q and k")
        if spec.dim > 256:
            raise ValueError(f"dim={spec.dim}: the memory kernel holds at most 256 rows per head")
        self.qk, self.vv = spec.qk_heads * spec.dim, spec.num_heads * spec.vdim
        self.conv_width = 2 * self.qk + self.vv
        # every segment of the fused product begins at a multiple of 8 columns
        self.a_at = _pad8(self.conv_width)
        self.g_at = self.a_at + _pad8(spec.decay_rank)
        self.b_at = self.g_at + _pad8(spec.gate_rank)
        self.cols = self.b_at + _pad8(spec.num_heads)
        q, kv = self.qk, 2 * self.qk
        self.conv = build_part("conv", CausalTapsSpec(
            self.conv_width, spec.taps, spec.q_conv_name, identity=False,
            weight_parts=((spec.q_conv_name, 0, q), (spec.k_conv_name, q, kv), (spec.v_conv_name, kv, self.conv_width))),
            prefix + ".conv", self.shared)
        self._conv_state = self.conv.cache_need()
        self._norm_rows: torch.Tensor | None = None
        # 32-bit numbers per token that the memory kernel prepares: q | k | decays | v | k.q | beta, in fours
        self._work_per_token = -(-(2 * self.qk + spec.num_heads * spec.dim + self.vv + spec.qk_heads + spec.num_heads) // 4) * 4

    def children(self) -> dict[str, Part]:
        return {"conv": self.conv}

    def cache_need(self):
        s: ChannelDeltaSpec = self.spec
        state = FixedState((s.num_heads, s.dim * s.vdim), "float32")
        return state if self._conv_state is None else (self._conv_state, state)

    def param_specs(self) -> dict[str, ParamSpec]:
        s: ChannelDeltaSpec = self.spec
        qk, vv = self.qk, self.vv
        return {
            "win": ParamSpec((self.cols, s.hidden), [
                Source(s.q_name, (0, qk)), Source(s.k_name, (qk, 2 * qk)), Source(s.v_name, (2 * qk, 2 * qk + vv)),
                Source(s.decay_in_name, (self.a_at, self.a_at + s.decay_rank)),
                Source(s.gate_in_name, (self.g_at, self.g_at + s.gate_rank)),
                Source(s.beta_name, (self.b_at, self.b_at + s.num_heads))]),
            "wa2": ParamSpec((s.num_heads * s.dim, s.decay_rank), [Source(s.decay_out_name)]),
            "wg2": ParamSpec((vv, s.gate_rank), [Source(s.gate_out_name)]),
            "dt_bias": ParamSpec((s.num_heads * s.dim,), [Source(s.decay_bias_name)], init="bias"),
            "a_log": ParamSpec((s.num_heads,), [Source(s.a_log_name)], init="bias"),
            "norm": ParamSpec((s.vdim,), [Source(s.norm_name)], init="ones"),
            "wo": ParamSpec((s.hidden, vv), [Source(s.o_name)]),
        }

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        super().bind(params)
        self._norm_rows = self.norm.repeat(self.spec.num_heads).contiguous()  # (the heads share one gain)

    def streamed_params(self) -> list[str]:
        return ["win", "wo"]

    def scratch_elements_per_token(self) -> int:
        s: ChannelDeltaSpec = self.spec
        return self.cols + 2 * s.num_heads * s.dim + 5 * self.vv + s.hidden + 2 * self._work_per_token

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        s: ChannelDeltaSpec = self.spec
        n, qk, vv, h = ctx.num_tokens, self.qk, self.vv, s.num_heads
        conv_cache, state = (None, cache) if self._conv_state is None else cache
        proj = ctx.scratch("delta_in", (n, self.cols), ctx.dtype)
        linear(x, self.win, None, proj, ctx.scratch)
        qkv = self.conv.forward(proj[:, :self.conv_width], ctx, conv_cache)
        g_raw = ctx.scratch("delta_decay", (n, h * s.dim), torch.float32)
        linear_f32_out(proj[:, self.a_at:self.a_at + s.decay_rank], self.wa2, g_raw)
        gate = ctx.scratch("delta_gate", (n, vv), ctx.dtype)
        linear(proj[:, self.g_at:self.g_at + s.gate_rank], self.wg2, None, gate, ctx.scratch)
        read = ctx.scratch("memory_read", (n, vv), torch.float32)
        work = ctx.scratch("delta_work", (n * self._work_per_token,), torch.float32)
        K.delta_recurrence(qkv[:, :qk], qkv[:, qk:2 * qk], qkv[:, 2 * qk:], proj[:, self.b_at:self.b_at + h], g_raw,
                           self.dt_bias, self.a_log, h, s.qk_heads, s.dim, s.vdim, state.state, state.slots,
                           ctx.cu_q, ctx.num_rows, read, act="silu", unit_eps=s.unit_eps, q_scale=s.dim ** -0.5,
                           work=work)
        gated = ctx.scratch("memory_gated", (n, vv), ctx.dtype)
        K.group_norm_gate(read, h, s.eps, self._norm_rows, gate, gated)
        y = ctx.scratch("memory_out", (n, s.hidden), ctx.dtype)
        return linear(gated, self.wo, None, y, ctx.scratch)
