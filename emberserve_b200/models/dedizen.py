"""Dedizen as an assembly of parts.

Every layer is a pre-norm block: ``x += mixer(norm1(x))``, then ``x += ff(norm2(x))`` where the layer
has a feed-forward (an ungated one with the square of relu).  The norms are plain RMS norms computed
in 32 bits.  The mixer is one of: ``parallel`` (chunked grouped-query attention with a sink, whose
values are its keys, beside linear attention with a fixed decay per head; the block takes the mean of
the two, each RMS-normed), ``mlstm`` (a matrix memory with exponential gates) or ``rglru`` (a gated
diagonal recurrence behind a short convolution).  The head is the embedding table.  Tensor names:
``embed``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``.
"""

from __future__ import annotations

from emberserve_b200.config.dedizen import (DedizenConfig, MLSTMConfig, ParallelMixerConfig, RGLRUConfig)
from emberserve_b200.parts.block import PreNormBlockSpec
from emberserve_b200.parts.decoder import DecoderSpec, LayerCall
from emberserve_b200.parts.mlp import DenseMLPSpec
from emberserve_b200.parts.norm import GroupedRMSNormSpec
from emberserve_b200.parts.parallel import ParallelMixersSpec
from emberserve_b200.parts.recurrent import DecayLinearAttentionSpec, MLSTMSpec, RGLRUSpec
from emberserve_b200.parts.rope import RotaryInterleavedSpec, RotaryYarnSpec
from emberserve_b200.parts.sink_attention import SinkAttentionSpec
from emberserve_b200.registry import register_architecture


def _mixer_spec(cfg: DedizenConfig, m, p: str):
    if isinstance(m, MLSTMConfig):
        return MLSTMSpec(hidden=cfg.width, num_heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap,
                         eps=cfg.norm_eps, q_name=p + "q", k_name=p + "k", v_name=p + "v", g_name=p + "g",
                         o_name=p + "o", norm_name=p + "norm", i_name=p + "i", i_bias_name=p + "i.b",
                         f_name=p + "f", f_bias_name=p + "f.b")
    if isinstance(m, RGLRUConfig):
        return RGLRUSpec(hidden=cfg.width, width=m.width, blocks=m.blocks, taps=m.conv, y_name=p + "y",
                         y_bias_name=p + "y.b", x_name=p + "x", x_bias_name=p + "x.b", conv_name=p + "conv",
                         conv_bias_name=p + "conv.b", ra_name=p + "ra", ra_bias_name=p + "ra.b", ri_name=p + "ri",
                         ri_bias_name=p + "ri.b", lam_name=p + "lam", o_name=p + "o")
    assert isinstance(m, ParallelMixerConfig)
    a, r = m.left, m.right
    position = None
    if a.rot_dims:
        if a.rot_scaling is not None:
            sc = a.rot_scaling
            position = RotaryYarnSpec(rotary_dim=a.rot_dims, theta=a.rot_base, max_positions=cfg.max_positions,
                                      factor=sc.factor, original=sc.original, fast=sc.fast, slow=sc.slow,
                                      pairing="interleaved")
        else:
            position = RotaryInterleavedSpec(rotary_dim=a.rot_dims, theta=a.rot_base,
                                             max_positions=cfg.max_positions)
    left = SinkAttentionSpec(
        hidden=cfg.width, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
        position=position, q_name=p + "left.q", k_name=p + "left.k", o_name=p + "left.o", v_name=None,
        q_bias_name=p + "left.q.b", k_bias_name=p + "left.k.b", sink_name=p + "left.sink",
        gate_name=p + "left.g", qk_norm_eps=cfg.norm_eps, chunk=a.chunk)
    right = DecayLinearAttentionSpec(
        hidden=cfg.width, num_heads=r.heads, dim=r.dim, vdim=r.vdim, decay=r.decay, eps=cfg.norm_eps,
        q_name=p + "right.q", k_name=p + "right.k", v_name=p + "right.v", g_name=p + "right.g",
        o_name=p + "right.o", norm_name=p + "right.norm", activation="silu")
    return ParallelMixersSpec(hidden=cfg.width, left=left, right=right, eps=cfg.norm_eps,
                              left_gain_name=p + "left.out", right_gain_name=p + "right.out")


def build_dedizen_spec(cfg: DedizenConfig) -> DecoderSpec:
    def norm(name: str) -> GroupedRMSNormSpec:
        return GroupedRMSNormSpec(cfg.width, 1, cfg.norm_eps, name)  # one group: the plain 32-bit RMS norm

    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}"
        ffn = None
        if L.mlp is not None:
            ffn = DenseMLPSpec(hidden=cfg.width, intermediate=L.mlp.ff, up_name=f"{p}.mlp.up",
                               down_name=f"{p}.mlp.down", activation="relu2")
        layers.append(PreNormBlockSpec(mixer=_mixer_spec(cfg, L.mixer, f"{p}.mix."), feed_forward=ffn,
                                       mixer_norm=norm(f"{p}.norm1"),
                                       ffn_norm=norm(f"{p}.norm2") if ffn is not None else None))
    # cache entries, in layer order: pages and a memory for a parallel mixer, one state for an mLSTM,
    # the convolution's inputs (with more than one tap) and the recurrence's state for an RG-LRU
    order, entry = [], 0
    for i, L in enumerate(cfg.layers):
        count = 1 if isinstance(L.mixer, MLSTMConfig) else 2
        if isinstance(L.mixer, RGLRUConfig) and L.mixer.conv == 1:
            count = 1
        ids = tuple(range(entry, entry + count))
        order.append(LayerCall(layer=i, cache=ids if count > 1 else ids[0]))
        entry += count
    return DecoderSpec(vocab_size=cfg.vocab_size, hidden=cfg.width, embed_name="embed", layers=layers, order=order,
                       final_norm=norm("final.norm"), head_name=None, max_positions=cfg.max_positions, ignorable=())


register_architecture("Dedizen", DedizenConfig, build_dedizen_spec)
