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
