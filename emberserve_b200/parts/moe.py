"""Routed experts: a feed-forward made of `num_experts` small gated feed-forwards, of which
every token uses `top_k`.

    z = Wr h                       router logits, 32-bit
    s = softmax(z)                 over ALL experts (`scoring` "sigmoid": sigmoid(z), each expert by itself)
    chosen = the top_k largest s   (ties: the lower index)
    weight = s[chosen]             as they are, or divided by their sum with `renormalize`
    y = sum_k weight_k * Wd[e_k] (act(Wg[e_k] h) * (Wu[e_k] h))
    y = sum_k Wd[e_k] glu(Wg[e_k] (weight_k h), Wu[e_k] (weight_k h))     with `weight_on_input`

With `shared_expert`, the spec of a dense feed-forward that every token uses, its output is added.
``RoutedMLP`` (below) is the form whose experts have no gate, with identity experts, a correction on the
choice and a constant on the weights.

The (token, choice) pairs are sorted by expert on the device and the experts run as two grouped
matrix products over the sorted rows (``csrc/moe_routed.cu``); nothing is read back to the host,
so the step can be captured in a CUDA graph.  A token's result is computed row by row and summed
over its choices in a fixed order: it does not depend on what else is in the step.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import FeedForward, ParamSpec, Part, Source, StepContext, build_part, register_part


# Steps of more tokens than this take the tcgen05 grouped product (the routing kernels lay the rows
# out for it only in their several-block form, above 512 tokens).
_GROUPED_TC05_TOKENS = 512


@dataclass(frozen=True)
class RoutedGLUSpec:
    hidden: int
    intermediate: int  # of one expert
    num_experts: int
    top_k: int
    router_name: str  # checkpoint tensor [num_experts, hidden]
    # per expert, the checkpoint tensors of its gate, up and down projections
    expert_names: tuple[tuple[str, str, str], ...]
    activation: str = "silu"  # one of kernels.GLU_ACTIVATIONS
    renormalize: bool = False
    kind: str = "routed_glu"
    scoring: str = "softmax"  # or "sigmoid"
    weight_on_input: bool = False  # the weight multiplies what the expert reads, not what it returns
    act_limit: float = 0.0  # the two constants of the activation "swiglu_capped"
    act_alpha: float = 1.0
    shared_expert: Any = None  # spec of a feed-forward that runs for every token and is added


@register_part("feed_forward", "routed_glu")
class RoutedGLU(FeedForward):
    router: torch.Tensor
    wgu: torch.Tensor  # [E * 2 ff, hidden]: per expert the gate rows, then the up rows
    wdown: torch.Tensor  # [E * hidden, ff]

    def __init__(self, spec: RoutedGLUSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if not 1 <= spec.top_k <= spec.num_experts:
            raise ValueError(f"top_k={spec.top_k} of {spec.num_experts} experts")
        if len(spec.expert_names) != spec.num_experts:
            raise ValueError("one (gate, up, down) name triple per expert is needed")
        if spec.activation not in K.GLU_ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r}: one of {sorted(K.GLU_ACTIVATIONS)}")
        if spec.scoring not in K.MOE_SCORINGS:
            raise ValueError(f"scoring {spec.scoring!r}: one of {sorted(K.MOE_SCORINGS)}")
        self._router32: torch.Tensor | None = None
        self.shared_ffn = (build_part("feed_forward", spec.shared_expert, prefix + ".shared", self.shared)
                           if spec.shared_expert is not None else None)

    def children(self) -> dict[str, Part]:
        return {} if self.shared_ffn is None else {"shared": self.shared_ffn}

    def param_specs(self) -> dict[str, ParamSpec]:
        s: RoutedGLUSpec = self.spec
        ff, hid = s.intermediate, s.hidden
        gu, down = [], []
        for e, (g, u, d) in enumerate(s.expert_names):
            gu += [Source(g, (2 * e * ff, (2 * e + 1) * ff)), Source(u, ((2 * e + 1) * ff, (2 * e + 2) * ff))]
            down.append(Source(d, (e * hid, (e + 1) * hid)))
        return {
            "router": ParamSpec((s.num_experts, hid), [Source(s.router_name)]),
            "wgu": ParamSpec((s.num_experts * 2 * ff, hid), gu),
            "wdown": ParamSpec((s.num_experts * hid, ff), down),
        }

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        super().bind(params)
        self._router32 = self.router.float()  # the logits are a 32-bit product

    def scratch_elements_per_token(self) -> int:
        s: RoutedGLUSpec = self.spec
        # activations of the chosen experts, their 32-bit outputs (two elements each), the result; in
        # prompt steps the gathered rows as well, and the padding of both to tiles of 256 rows
        return 2 * s.top_k * (s.intermediate + 2 * s.hidden) + 3 * s.hidden + (s.hidden if s.shared_expert else 0)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        s: RoutedGLUSpec = self.spec
        n, e, top = x.shape[0], s.num_experts, s.top_k
        pairs = n * top
        x32 = x
        if x.dtype != torch.float32:
            x32 = ctx.scratch("moe_x32", (n, s.hidden), torch.float32)
            x32.copy_(x)
        logits = ctx.scratch("moe_logits", (n, e), torch.float32)
        torch.mm(x32, self._router32.t(), out=logits)
        tile = K.moe_tile_rows()
        max_tiles = K.moe_max_tiles(pairs, e, tile)
        ids = ctx.scratch("moe_ids", (pairs,), torch.int32)
        weights = ctx.scratch("moe_weights", (pairs,), torch.float32)
        offsets = ctx.scratch("moe_offsets", (3 * e + 1,), torch.int32)
        plan = ctx.scratch("moe_plan", (1 + 3 * max_tiles,), torch.int32)
        wgu = self.wgu.view(e, 2 * s.intermediate, s.hidden)
        # Prompt steps in bfloat16: every expert's sorted rows start at a multiple of 256, the rows are
        # gathered into that layout, and the gate/up product runs on the two-SM tcgen05 kernel in its
        # grouped form (the down product reads the same layout through the tile list).
        extra = None
        if self.shared_ffn is not None:
            # (its result stays in a buffer of its own until the routed experts' sum takes it in)
            extra = ctx.scratch("ffn_shared", (n, s.hidden), ctx.dtype)
            extra.copy_(self.shared_ffn.forward(x, ctx))
        scaled_in = weights if s.weight_on_input else None
        if (x.is_cuda and ctx.dtype == torch.bfloat16 and n > _GROUPED_TC05_TOKENS
                and s.activation in ("silu", "swiglu_capped")
                and K.moe_up_grouped_tc05_supported(s.intermediate, s.hidden)):
            big_rows = K.MOE_BIG_TILE_ROWS
            big = ctx.scratch("moe_big", (K.moe_max_tiles(pairs, e, big_rows),), torch.int32)
            rows = big.numel() * big_rows
            perm = ctx.scratch("moe_perm", (rows,), torch.int32)
            inv = ctx.scratch("moe_inv", (pairs,), torch.int32)
            K.moe_route(logits, top, s.renormalize, ids, weights, offsets, perm, plan, max_tiles, align=big_rows,
                        big=big, inv=inv, scoring=s.scoring)
            xs = ctx.scratch("moe_xs", (rows, s.hidden), ctx.dtype)
            K.moe_gather(x, perm, top, xs)
            act = ctx.scratch("moe_act", (rows, s.intermediate), ctx.dtype)
            K.moe_up_grouped_tc05(xs, wgu, big, act, s.activation, perm, scaled_in, s.act_limit, s.act_alpha)
            if s.intermediate % 8 == 0 and s.hidden % 8 == 0:  # the down product in the same form
                y16 = ctx.scratch("moe_y16", (rows, s.hidden), ctx.dtype)
                K.moe_down_grouped_tc05(act, self.wdown.view(e, s.hidden, s.intermediate), big, y16)
                out = ctx.scratch("ffn_out", (n, s.hidden), ctx.dtype)
                K.moe_combine_rows(y16, inv, None if s.weight_on_input else weights, out, top, extra=extra)
                return out
        else:
            perm = ctx.scratch("moe_perm", (pairs,), torch.int32)
            K.moe_route(logits, top, s.renormalize, ids, weights, offsets, perm, plan, max_tiles, scoring=s.scoring)
            act = ctx.scratch("moe_act", (pairs, s.intermediate), ctx.dtype)
            K.moe_up(x, wgu, perm, offsets, plan, max_tiles, top, s.activation, act, in_scale=scaled_in,
                     limit=s.act_limit, alpha=s.act_alpha)
        y = ctx.scratch("moe_y", (pairs, s.hidden), torch.float32)
        K.moe_down(act, self.wdown.view(e, s.hidden, s.intermediate), perm, offsets, plan, max_tiles, y)
        out = ctx.scratch("ffn_out", (n, s.hidden), ctx.dtype)
        K.moe_combine(y, None if s.weight_on_input else weights, out, top, extra=extra)
        return out


@dataclass(frozen=True)
class RoutedMLPSpec:
    hidden: int
    intermediate: int  # of one expert
    num_experts: int  # experts with weights
    top_k: int
    router_name: str  # checkpoint tensor [num_experts + identity_experts, hidden]
    expert_names: tuple[tuple[str, str], ...]  # per expert with weights, its up and down projections
    activation: str = "gelu"  # one of kernels.EXPERT_ACTIVATIONS
    identity_experts: int = 0  # further router outputs whose expert returns its input
    correction_name: str | None = None  # [num_experts + identity_experts]: added to the scores for the choice only
    renormalize: bool = True  # the chosen scores are divided by (their sum + renorm_eps)
    renorm_eps: float = 1e-20
    route_scale: float = 1.0  # multiplies the weights
    shared_expert: Any = None  # spec of a feed-forward that runs for every token and is added
    kind: str = "routed_mlp"


@register_part("feed_forward", "routed_mlp")
class RoutedMLP(FeedForward):
    """Routed experts without a gate: ``expert_e(h) = Wd[e] act(Wu[e] h)``.

        z = Wr h                      router logits over the experts AND the identity experts, 32-bit
        s = softmax(z)
        chosen = the top_k largest of s + correction       (the weights use s alone)
        weight = s[chosen] / (sum + renorm_eps) * route_scale
        y = sum_k weight_k * (h if e_k is an identity expert else expert_(e_k)(h))  (+ shared expert)

    Routing, the sort by expert, the two grouped products and the combine step are the kernels of
    ``RoutedGLU`` (``csrc/moe_routed.cu``) in their ungated form; identity experts get no tiles and the
    combine step adds the token's own input for them."""

    router: torch.Tensor
    wup: torch.Tensor  # [E * ff, hidden]
    wdown: torch.Tensor  # [E * hidden, ff]
    correction: torch.Tensor | None = None

    def __init__(self, spec: RoutedMLPSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        self.total = spec.num_experts + spec.identity_experts
        if spec.num_experts < 1 or spec.identity_experts < 0 or not 1 <= spec.top_k <= self.total:
            raise ValueError(f"top_k={spec.top_k} of {spec.num_experts} experts and {spec.identity_experts} "
                             f"identity experts")
        if len(spec.expert_names) != spec.num_experts:
            raise ValueError("one (up, down) name pair per expert is needed")
        if spec.activation not in K.EXPERT_ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r}: one of {sorted(K.EXPERT_ACTIVATIONS)}")
        self._router32: torch.Tensor | None = None
        self._correction32: torch.Tensor | None = None
        self.shared_ffn = (build_part("feed_forward", spec.shared_expert, prefix + ".shared", self.shared)
                           if spec.shared_expert is not None else None)

    def children(self) -> dict[str, Part]:
        return {} if self.shared_ffn is None else {"shared": self.shared_ffn}

    def param_specs(self) -> dict[str, ParamSpec]:
        s: RoutedMLPSpec = self.spec
        ff, hid = s.intermediate, s.hidden
        specs = {
            "router": ParamSpec((self.total, hid), [Source(s.router_name)]),
            "wup": ParamSpec((s.num_experts * ff, hid),
                             [Source(u, (e * ff, (e + 1) * ff)) for e, (u, _) in enumerate(s.expert_names)]),
            "wdown": ParamSpec((s.num_experts * hid, ff),
                               [Source(d, (e * hid, (e + 1) * hid)) for e, (_, d) in enumerate(s.expert_names)]),
        }
        if s.correction_name is not None:
            specs["correction"] = ParamSpec((self.total,), [Source(s.correction_name)], init="bias")
        return specs

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        super().bind(params)
        self._router32 = self.router.float()  # the logits are a 32-bit product
        self._correction32 = None if self.correction is None else self.correction.float().contiguous()

    def scratch_elements_per_token(self) -> int:
        s: RoutedMLPSpec = self.spec
        # activations of the chosen experts, their 32-bit outputs (two elements each), the result; in prompt
        # steps the gathered rows as well, and the padding of both to tiles of 256 rows
        return 2 * s.top_k * (s.intermediate + 2 * s.hidden) + 4 * s.hidden + 2 * self.total

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        s: RoutedMLPSpec = self.spec
        n, e, top = x.shape[0], self.total, s.top_k
        pairs = n * top
        x32 = x
        if x.dtype != torch.float32:
            x32 = ctx.scratch("moe_x32", (n, s.hidden), torch.float32)
            x32.copy_(x)
        logits = ctx.scratch("moe_logits", (n, e), torch.float32)
        torch.mm(x32, self._router32.t(), out=logits)
        tile = K.moe_tile_rows()
        max_tiles = K.moe_max_tiles(pairs, e, tile)
        ids = ctx.scratch("moe_ids", (pairs,), torch.int32)
        weights = ctx.scratch("moe_weights", (pairs,), torch.float32)
        offsets = ctx.scratch("moe_offsets", (3 * e + 1,), torch.int32)
        plan = ctx.scratch("moe_plan", (1 + 3 * max_tiles,), torch.int32)
        perm = ctx.scratch("moe_perm", (pairs,), torch.int32)
        extra = None
        if self.shared_ffn is not None:
            # (its result stays in a buffer of its own until the routed experts' sum takes it in)
            extra = ctx.scratch("ffn_shared", (n, s.hidden), ctx.dtype)
            extra.copy_(self.shared_ffn.forward(x, ctx))
        routing = dict(correction=self._correction32, renorm_eps=s.renorm_eps, scale=s.route_scale,
                       plan_experts=s.num_experts)
        same = dict(ids=ids, x=x, num_real=s.num_experts) if s.identity_experts else {}
        if (x.is_cuda and ctx.dtype == torch.bfloat16 and n > _GROUPED_TC05_TOKENS and s.intermediate % 8 == 0
                and s.hidden % 8 == 0):
            # Prompt steps in bfloat16: every expert's sorted rows start at a multiple of 256, the rows are
            # gathered into that layout and both products run on the grouped tcgen05 kernel (groups of
            # identity experts belong to nobody and are skipped); the activation is a pass of its own.
            big_rows = K.MOE_BIG_TILE_ROWS
            big = ctx.scratch("moe_big", (K.moe_max_tiles(pairs, e, big_rows),), torch.int32)
            rows = big.numel() * big_rows
            perm = ctx.scratch("moe_perm", (rows,), torch.int32)
            inv = ctx.scratch("moe_inv", (pairs,), torch.int32)
            K.moe_route(logits, top, s.renormalize, ids, weights, offsets, perm, plan, max_tiles, align=big_rows,
                        big=big, inv=inv, **routing)
            xs = ctx.scratch("moe_xs", (rows, s.hidden), ctx.dtype)
            K.moe_gather(x, perm, top, xs)
            act = ctx.scratch("moe_act", (rows, s.intermediate), ctx.dtype)
            K.moe_down_grouped_tc05(xs, self.wup.view(s.num_experts, s.intermediate, s.hidden), big, act)
            K.unary_act(act, act, s.activation)
            y16 = ctx.scratch("moe_y16", (rows, s.hidden), ctx.dtype)
            K.moe_down_grouped_tc05(act, self.wdown.view(s.num_experts, s.hidden, s.intermediate), big, y16)
            out = ctx.scratch("ffn_out", (n, s.hidden), ctx.dtype)
            K.moe_combine_rows(y16, inv, weights, out, top, extra=extra, **same)
            return out
        K.moe_route(logits, top, s.renormalize, ids, weights, offsets, perm, plan, max_tiles, **routing)
        act = ctx.scratch("moe_act", (pairs, s.intermediate), ctx.dtype)
        K.moe_up(x, self.wup.view(s.num_experts, s.intermediate, s.hidden), perm, offsets, plan, max_tiles, top,
                 s.activation, act, gated=False)
        y = ctx.scratch("moe_y", (pairs, s.hidden), torch.float32)
        K.moe_down(act, self.wdown.view(s.num_experts, s.hidden, s.intermediate), perm, offsets, plan, max_tiles, y)
        out = ctx.scratch("ffn_out", (n, s.hidden), ctx.dtype)
        K.moe_combine(y, weights, out, top, extra=extra, **same)
        return out
