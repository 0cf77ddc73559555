"""Damolorn as an assembly of parts.

Every layer is a sandwich block (a grouped RMSNorm before and behind each sub-layer) whose mixer
reads its input through a short causal convolution.  The mixer is latent attention in one of two
variants: ``latent_attention`` (rotate-half pairing of the rotated part, a sigmoid output gate)
and ``latent_attention_2`` (interleaved pairing, no gate).  The feed-forward is a dense gated one
with ReLU, routed SiLU-gated experts whose weights are the softmax scores as they are, or absent.
A range of layers may run several times with the same weights; each run has cache entries of its
own, and each pass begins by adding a vector of ``loop.step`` (and, from the second pass on, the
embedding once more) to the stream.  Tensor names: ``embed``, ``head``, ``final.norm``,
``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b|canon1``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from emberserve_b200.config.damolorn import DamolornConfig
from emberserve_b200.parts.block import SandwichBlockSpec
from emberserve_b200.parts.conv import CausalTapsSpec
from emberserve_b200.parts.decoder import DecoderSpec, LayerCall, StreamInject
from emberserve_b200.parts.latent_attention import LatentAttentionSpec
from emberserve_b200.parts.mlp import SwiGLUSpec
from emberserve_b200.parts.moe import RoutedGLUSpec
from emberserve_b200.parts.norm import GroupedRMSNormSpec
from emberserve_b200.parts.rope import RotaryInterleavedSpec, RotarySpec
from emberserve_b200.registry import register_architecture


def build_damolorn_spec(cfg: DamolornConfig) -> DecoderSpec:
    def norm(name: str) -> GroupedRMSNormSpec:
        return GroupedRMSNormSpec(cfg.width, cfg.norm_groups, cfg.norm_eps, name)

    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        gated = L.type == "latent_attention"
        position = None
        if m.rot_dims:
            rotary = RotarySpec if L.type == "latent_attention" else RotaryInterleavedSpec
            position = rotary(rotary_dim=m.rot_dims, theta=m.rot_base, max_positions=cfg.max_positions)
        mixer = LatentAttentionSpec(
            hidden=cfg.width, num_heads=m.heads, nope_dim=m.dim, rope_dim=m.rot_dim, v_dim=m.vdim,
            kv_rank=m.kv_rank, q_rank=m.q_rank, eps=cfg.norm_eps, scale=m.scale, position=position, gated=gated,
            dq_name=f"{p}.mix.dq", dq_norm_name=f"{p}.mix.dq.norm", uq_name=f"{p}.mix.uq",
            dkv_name=f"{p}.mix.dkv", dkv_norm_name=f"{p}.mix.dkv.norm", uk_name=f"{p}.mix.uk",
            uv_name=f"{p}.mix.uv", o_name=f"{p}.mix.o", g_name=f"{p}.mix.g" if gated else None)
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = SwiGLUSpec(hidden=cfg.width, intermediate=L.mlp.ff, gate_name=f"{p}.mlp.gate",
                             up_name=f"{p}.mlp.up", down_name=f"{p}.mlp.down", activation="relu", weight_suffix="")
        elif L.mlp is not None:
            ffn = RoutedGLUSpec(
                hidden=cfg.width, intermediate=L.mlp.ff, num_experts=L.mlp.experts, top_k=L.mlp.top,
                router_name=f"{p}.mlp.router",
                expert_names=tuple((f"{p}.mlp.e{e}.gate", f"{p}.mlp.e{e}.up", f"{p}.mlp.e{e}.down")
                                   for e in range(L.mlp.experts)),
                activation="silu", renormalize=False)
        layers.append(SandwichBlockSpec(
            mixer=mixer, mixer_norm=norm(f"{p}.norm1"), mixer_post_norm=norm(f"{p}.norm1b"),
            feed_forward=ffn, ffn_norm=norm(f"{p}.norm2") if ffn is not None else None,
            ffn_post_norm=norm(f"{p}.norm2b") if ffn is not None else None,
            mixer_conv=CausalTapsSpec(cfg.width, cfg.canon_taps, f"{p}.canon1") if cfg.canon_taps else None))
    has_state = cfg.canon_taps > 1
    order = []
    for run, (i, begins) in enumerate(cfg.layer_runs()):
        inject = None
        if begins is not None:
            inject = StreamInject(embedding=begins > 0, table="loop_step", row=begins)
        cache = (2 * run, 2 * run + 1) if has_state else run
        order.append(LayerCall(layer=i, cache=cache, inject=inject))
    return DecoderSpec(
        vocab_size=cfg.vocab_size, hidden=cfg.width, embed_name="embed", layers=layers, order=order,
        final_norm=norm("final.norm"), head_name="head", max_positions=cfg.max_positions, ignorable=(),
        tables={"loop_step": ("loop.step", cfg.loop_times)} if cfg.has_loop else {})


register_architecture("Damolorn", DamolornConfig, build_damolorn_spec)
