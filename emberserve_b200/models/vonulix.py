"""Vonulix as an assembly of parts.

The embedding row is scaled as it enters the 32-bit stream.  Every layer is a pre-norm block whose
norms store their gain minus one: ``x += mixer(norm1(x))``, then ``x += ff(norm2(x))`` where the
layer has a feed-forward.  The mixer is grouped-query attention with a linearly scaled partial
rotation of q and k, unit-RMS values that are turned by their own position before they are cached
(the sum over the values is turned back by the query's position), a window that also keeps the first
keys, and a sigmoid gate per head.  The feed-forward is a mixture of capped gated experts chosen by
sigmoid scores that multiply the expert's input, beside an optional shared expert with a sigmoid gate
per token.  Behind the sub-layers a layer adds an input of its own from a second embedding table
(where the model has one) and hands on a weighted sum of the stream's states at all depths so far.
Tensor names: ``embed``, ``head``, ``final.norm``, ``side.embed``, ``l<i>.norm1|norm2``,
``l<i>.mix.q|k|v|g|o``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down|sg``, ``l<i>.side.gate|proj|norm``, ``l<i>.dwa``.
"""

from __future__ import annotations

from emberserve_b200.config.vonulix import EXPERT_ACT_ALPHA, VonulixConfig
from emberserve_b200.parts.block import PreNormBlockSpec
from emberserve_b200.parts.decoder import DecoderSpec, LayerCall
from emberserve_b200.parts.mlp import SwiGLUSpec
from emberserve_b200.parts.moe import RoutedGLUSpec
from emberserve_b200.parts.norm import GroupedRMSNormSpec
from emberserve_b200.parts.rope import RotaryLinearSpec
from emberserve_b200.parts.sink_attention import SinkAttentionSpec
from emberserve_b200.parts.stream import DepthAverageSpec, TokenSideInputSpec, TokenTableSpec
from emberserve_b200.registry import register_architecture


def _mixer_spec(cfg: VonulixConfig, m, p: str) -> SinkAttentionSpec:
    position = None
    if m.rot_dims:
        position = RotaryLinearSpec(rotary_dim=m.rot_dims, theta=m.rot_base, max_positions=cfg.max_positions,
                                    factor=m.rot_factor)
    # the values turn over their whole length, at the keys' base and without the keys' scaling
    value_position = RotaryLinearSpec(rotary_dim=m.vdim, theta=m.rot_base, max_positions=cfg.max_positions)
    return SinkAttentionSpec(
        hidden=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale,
        position=position, q_name=p + "q", k_name=p + "k", v_name=p + "v", o_name=p + "o", gate_name=p + "g",
        window=m.window, keep_first=m.keep_first, v_head_dim=m.vdim, v_norm_eps=cfg.norm_eps,
        value_position=value_position)


def _ffn_spec(cfg: VonulixConfig, m, p: str) -> RoutedGLUSpec:
    shared = None
    if m.shared is not None:
        q = p + "shared."
        shared = SwiGLUSpec(hidden=cfg.width, intermediate=m.shared.ff, gate_name=q + "gate", up_name=q + "up",
                            down_name=q + "down", activation="swiglu_capped", weight_suffix="",
                            act_limit=m.shared.limit, act_alpha=EXPERT_ACT_ALPHA, token_gate_name=q + "sg")
    return RoutedGLUSpec(
        hidden=cfg.width, intermediate=m.expert.ff, num_experts=m.experts, top_k=m.top, router_name=p + "router",
        expert_names=tuple((f"{p}e{j}.gate", f"{p}e{j}.up", f"{p}e{j}.down") for j in range(m.experts)),
        activation="swiglu_capped", scoring="sigmoid", weight_on_input=True, act_limit=m.expert.limit,
        act_alpha=EXPERT_ACT_ALPHA, shared_expert=shared)


def build_vonulix_spec(cfg: VonulixConfig) -> DecoderSpec:
    def norm(name: str) -> GroupedRMSNormSpec:
        # one group: the plain 32-bit RMS norm; the stored weight is the gain minus one
        return GroupedRMSNormSpec(cfg.width, 1, cfg.norm_eps, name, gain_offset=1.0)

    depths = len(cfg.layers)
    table = (TokenTableSpec(vocab_size=cfg.vocab_size, width=depths * cfg.side_dim, name="side.embed")
             if cfg.side_dim else None)
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}"
        ffn = _ffn_spec(cfg, L.mlp, f"{p}.mlp.") if L.mlp is not None else None
        stream = []
        if table is not None:
            stream.append(TokenSideInputSpec(hidden=cfg.width, dim=cfg.side_dim, column=i * cfg.side_dim,
                                             table=table, eps=cfg.norm_eps, gate_name=f"{p}.side.gate",
                                             proj_name=f"{p}.side.proj", norm_name=f"{p}.side.norm"))
        stream.append(DepthAverageSpec(hidden=cfg.width, depth=i, depths=depths, weight_name=f"{p}.dwa"))
        layers.append(PreNormBlockSpec(mixer=_mixer_spec(cfg, L.mixer, f"{p}.mix."), feed_forward=ffn,
                                       mixer_norm=norm(f"{p}.norm1"),
                                       ffn_norm=norm(f"{p}.norm2") if ffn is not None else None,
                                       stream_parts=tuple(stream)))
    order = [LayerCall(layer=i, cache=i) for i in range(depths)]
    return DecoderSpec(vocab_size=cfg.vocab_size, hidden=cfg.width, embed_name="embed", layers=layers, order=order,
                       final_norm=norm("final.norm"), head_name="head", max_positions=cfg.max_positions,
                       ignorable=(), embed_scale=cfg.embed_scale)


register_architecture("Vonulix", VonulixConfig, build_vonulix_spec)
