"""Lesosun as an assembly of parts.

The embedding is RMS-normed; every layer adds ``m * (mixer(norm1(x)) + ff(norm2(x)))`` to the stream,
both norms taken of the same x (their gains are stored minus one); the mixer is ``parallel`` (grouped-query
attention behind short convolutions, with normed and rotated q and k and capped scores, beside a
selective state space; the two are summed with weights) or ``channel_delta`` (the delta rule with a decay
per key channel); the feed-forward is a SiLU-gated dense one, routed ungated experts (with identity
experts, a correction on the choice and an optional shared expert) or absent.  The head is the embedding
table and the logits are capped.  Tensor names: ``embed``, ``embed.norm``, ``final.norm``,
``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from emberserve_b200.config.lesosun import ChannelDeltaConfig, FeedForwardConfig, LesosunConfig, ParallelMixerConfig
from emberserve_b200.config.model import ConfigError
from emberserve_b200.parts.block import SharedInputBlockSpec
from emberserve_b200.parts.decoder import DecoderSpec, LayerCall
from emberserve_b200.parts.mlp import DenseMLPSpec, SwiGLUSpec
from emberserve_b200.parts.moe import RoutedMLPSpec
from emberserve_b200.parts.norm import GroupedRMSNormSpec
from emberserve_b200.parts.parallel import ParallelMixersSpec
from emberserve_b200.parts.recurrent import ChannelDeltaSpec, SelectiveStateSpaceSpec
from emberserve_b200.parts.rope import RotaryInterleavedSpec
from emberserve_b200.parts.sink_attention import SinkAttentionSpec
from emberserve_b200.registry import register_architecture


def _mixer_spec(cfg: LesosunConfig, m, p: str, where: str):
    if isinstance(m, ChannelDeltaConfig):
        if m.decay_rank is None or m.gate_rank is None:
            raise ConfigError(f"{where}: the inner sizes of the decay and gate projections are given by the "
                              f"checkpoint's tensors {p}a1 and {p}g1 (or by decay_rank / gate_rank in the file)")
        return ChannelDeltaSpec(
            hidden=cfg.width, num_heads=m.heads, qk_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, taps=m.conv,
            decay_rank=m.decay_rank, gate_rank=m.gate_rank, eps=cfg.norm_eps, q_name=p + "q", k_name=p + "k",
            v_name=p + "v", q_conv_name=p + "q.conv", k_conv_name=p + "k.conv", v_conv_name=p + "v.conv",
            beta_name=p + "b", a_log_name=p + "A_log", decay_in_name=p + "a1", decay_out_name=p + "a2",
            decay_bias_name=p + "dt_bias", gate_in_name=p + "g1", gate_out_name=p + "g2", norm_name=p + "norm",
            o_name=p + "o")
    assert isinstance(m, ParallelMixerConfig)
    a, r = m.left, m.right
    position = (RotaryInterleavedSpec(rotary_dim=a.rot_dims, theta=a.rot_base, max_positions=cfg.max_positions)
                if a.rot_dims else None)
    q = p + "left."
    left = SinkAttentionSpec(
        hidden=cfg.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
        position=position, q_name=q + "q", k_name=q + "k", o_name=q + "o", v_name=q + "v", q_bias_name=q + "q.b",
        k_bias_name=q + "k.b", v_bias_name=q + "v.b", qk_norm_eps=cfg.norm_eps,
        v_head_dim=None if a.vdim == a.dim else a.vdim, conv_taps=a.conv, q_conv_name=q + "q.conv",
        k_conv_name=q + "k.conv", v_conv_name=q + "v.conv", q_norm_name=q + "q.norm", k_norm_name=q + "k.norm",
        norm_before_rotation=True, softcap=a.softcap, o_bias_name=q + "o.b")
    q = p + "right."
    right = SelectiveStateSpaceSpec(
        hidden=cfg.width, num_heads=r.heads, vdim=r.vdim, state=r.state, groups=r.groups, norm_groups=r.norm_groups,
        taps=r.conv, eps=cfg.norm_eps, in_name=q + "in", conv_name=q + "conv", conv_bias_name=q + "conv.b",
        dt_bias_name=q + "dt_bias", a_log_name=q + "A_log", d_name=q + "D", norm_name=q + "norm", o_name=q + "o")
    return ParallelMixersSpec(hidden=cfg.width, left=left, right=right, combine="weighted",
                              left_scale=m.left_scale, right_scale=m.right_scale)


def _ffn_spec(cfg: LesosunConfig, f: FeedForwardConfig, p: str):
    if f.kind == "dense":
        return SwiGLUSpec(hidden=cfg.width, intermediate=f.ff, gate_name=p + "gate", up_name=p + "up",
                          down_name=p + "down", weight_suffix="")
    shared = None
    if f.shared_ff is not None:
        shared = DenseMLPSpec(hidden=cfg.width, intermediate=f.shared_ff, up_name=p + "shared.up",
                              down_name=p + "shared.down", activation="gelu")
    return RoutedMLPSpec(hidden=cfg.width, intermediate=f.ff, num_experts=f.experts, top_k=f.top,
                         router_name=p + "router",
                         expert_names=tuple((f"{p}e{e}.up", f"{p}e{e}.down") for e in range(f.experts)),
                         activation="gelu", identity_experts=f.identity, correction_name=p + "correction",
                         renormalize=True, renorm_eps=1e-20, route_scale=f.route_scale, shared_expert=shared)


def build_lesosun_spec(cfg: LesosunConfig) -> DecoderSpec:
    def norm(name: str) -> GroupedRMSNormSpec:
        return GroupedRMSNormSpec(cfg.width, 1, cfg.norm_eps, name, gain_offset=1.0)  # gains stored minus one

    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}"
        ffn = None if L.mlp is None else _ffn_spec(cfg, L.mlp, f"{p}.mlp.")
        layers.append(SharedInputBlockSpec(mixer=_mixer_spec(cfg, L.mixer, f"{p}.mix.", f"layers[{i}].mixer"),
                                           mixer_norm=norm(f"{p}.norm1"), feed_forward=ffn,
                                           ffn_norm=norm(f"{p}.norm2") if ffn is not None else None,
                                           residual_mult=cfg.residual_mult))
    # cache entries, in layer order.  parallel: pages of the attention, its convolution's inputs, the state
    # space's convolution inputs, its state; channel_delta: the convolution's inputs and the memory
    # (a convolution of one tap keeps nothing)
    order, entry = [], 0
    for i, L in enumerate(cfg.layers):
        if isinstance(L.mixer, ChannelDeltaConfig):
            count = 1 + (L.mixer.conv > 1)
        else:
            count = 2 + (L.mixer.left.conv > 1) + (L.mixer.right.conv > 1)
        ids = tuple(range(entry, entry + count))
        order.append(LayerCall(layer=i, cache=ids if count > 1 else ids[0]))
        entry += count
    return DecoderSpec(vocab_size=cfg.vocab_size, hidden=cfg.width, embed_name="embed", layers=layers, order=order,
                       final_norm=norm("final.norm"), head_name=None, max_positions=cfg.max_positions, ignorable=(),
                       embed_norm=norm("embed.norm"), logit_softcap=cfg.logit_softcap)


register_architecture("Lesosun", LesosunConfig, build_lesosun_spec)
