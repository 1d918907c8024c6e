"""Routed experts: a feed-forward made of `num_experts` small gated feed-forwards, of which
every token uses `top_k`.

    z = Wr h                       router logits, 32-bit
    s = softmax(z)                 over ALL experts (`scoring` "sigmoid": sigmoid(z), each expert by itself)
    chosen = the top_k largest s   (ties: the lower index)
    weight = s[chosen]             as they are, or divided by their sum with `renormalize`
    y = sum_k weight_k * Wd[e_k] (act(Wg[e_k] h) * (Wu[e_k] h))
    y = sum_k Wd[e_k] glu(Wg[e_k] (weight_k h), Wu[e_k] (weight_k h))     with `weight_on_input`

With `shared_expert`, the spec of a dense feed-forward that every token uses, its output is added.

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
