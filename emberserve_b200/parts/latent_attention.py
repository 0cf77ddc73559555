"""Latent attention: queries, keys and values all pass through low-rank latents, and only the
key/value latent and one rotated key part shared by all heads are cached.

Per token, with input h::

    cq = RMSNorm(Wdq h) * gq                       query latent, q_rank numbers
    q  = Wuq cq                                    per head [plain (nope_dim) | rotated (rope_dim)]
    [kv | kr] = Wdkv h ;  c = RMSNorm(kv) * gkv    key/value latent, kv_rank numbers
    krot = rotate(kr)                              rope_dim numbers, one for all heads
    k_plain[h] = Wuk[h] c ,  v[h] = Wuv[h] c
    score(i, j, h) = (q_plain[i, h] . k_plain[j, h] + rotate(q_rot[i, h]) . krot[j]) * scale
    o[i, h] = sum_j softmax_j(score(i, :, h)) v[j, h]             (causal)
    y = Wo (o * sigmoid(Wg h))                     the gate only if the spec has one

The cache holds ``[c | krot]`` per token (``PagedLatent(kv_rank + rope_dim)``).  Because
k_plain and v are linear in c, the step computes ``qlat[h] = q_plain[h] Wuk[h]`` (the key
up-projection folded into the query), attends over the cached vectors themselves
(``csrc/latent_attention.cu``) and applies Wuv[h] to the attended latent; prompt portions and
single decoded tokens take the same path, so a token's result does not depend on how its
request was cut into steps.  Down-projections of query and key/value (and the gate) are one
matrix product; the per-head products are batched ones in the vendor library.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (Mixer, PagedLatent, PagedLatentHandle, ParamSpec, Source, StepContext,
                                        register_part)
from emberserve_b200.parts.linear import linear

# Keys of a token are cut over several blocks when a step has too few tokens to fill the device.
# One block per SM is the aim: at real sizes (512 + 64 numbers per key) a block's two tiles of keys
# take most of an SM's shared memory (64 rows at 2048 keys: 73 us with 128 blocks, 81 with 256).
_BLOCKS_PER_SM = 1
_MAX_SPLITS = 64
_MIN_KEYS_PER_SPLIT = 128


@dataclass(frozen=True)
class LatentAttentionSpec:
    hidden: int
    num_heads: int
    nope_dim: int  # query/key numbers per head that are not rotated
    rope_dim: int  # rotated query numbers per head = size of the shared key part
    v_dim: int
    kv_rank: int
    q_rank: int
    eps: float  # of the two latent RMSNorms
    scale: float
    position: Any  # rotary spec ("rotary_neox" or "rotary_interleaved"); its rotary_dim <= rope_dim
    gated: bool
    # checkpoint tensors
    dq_name: str
    dq_norm_name: str
    uq_name: str
    dkv_name: str
    dkv_norm_name: str
    uk_name: str
    uv_name: str
    o_name: str
    g_name: str | None = None
    window: int | None = None
    kind: str = "latent_attention"


def latent_splits(num_tokens: int, head_chunks: int, max_ctx: int, sms: int | None = None) -> int:
    """Over how many blocks the keys of one token are cut: a function of shapes and of the
    device's SM count only."""
    blocks = max(1, num_tokens * head_chunks)
    target = _BLOCKS_PER_SM * (sms if sms is not None else K.sm_count())
    cap = max(1, max_ctx // _MIN_KEYS_PER_SPLIT)
    return max(1, min(_MAX_SPLITS, target // blocks, cap))


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    w_in: torch.Tensor
    q_gain: torch.Tensor
    kv_gain: torch.Tensor
    wuq: torch.Tensor
    wuk: torch.Tensor
    wuv: torch.Tensor
    wo: torch.Tensor

    def __init__(self, spec: LatentAttentionSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        for name in ("num_heads", "nope_dim", "v_dim", "kv_rank", "q_rank"):
            if getattr(spec, name) <= 0:
                raise ValueError(f"{name} must be positive, got {getattr(spec, name)}")
        if spec.rope_dim < 0 or (spec.gated and spec.g_name is None):
            raise ValueError("latent attention: rope_dim must not be negative; a gate needs its tensor")
        if spec.kv_rank > 512:
            raise ValueError(f"kv_rank={spec.kv_rank}: the latent attention kernel takes up to 512")
        self.position = self.shared.get("position", spec.position) if spec.position is not None else None
        self.rot_dims = spec.position.rotary_dim if spec.position is not None else 0
        if self.rot_dims > spec.rope_dim:
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit into rope_dim={spec.rope_dim}")
        self.q_head = spec.nope_dim + spec.rope_dim
        self.in_rows = spec.q_rank + spec.kv_rank + spec.rope_dim + (spec.num_heads * spec.v_dim if spec.gated else 0)

    def cache_need(self) -> PagedLatent:
        s: LatentAttentionSpec = self.spec
        return PagedLatent(s.kv_rank + s.rope_dim, s.window)

    def param_specs(self) -> dict[str, ParamSpec]:
        s: LatentAttentionSpec = self.spec
        a, b = s.q_rank, s.q_rank + s.kv_rank + s.rope_dim
        rows = [Source(s.dq_name, (0, a)), Source(s.dkv_name, (a, b))]
        if s.gated:
            rows.append(Source(s.g_name, (b, self.in_rows)))
        return {
            "w_in": ParamSpec((self.in_rows, s.hidden), rows),
            "q_gain": ParamSpec((s.q_rank,), [Source(s.dq_norm_name)], init="ones"),
            "kv_gain": ParamSpec((s.kv_rank,), [Source(s.dkv_norm_name)], init="ones"),
            "wuq": ParamSpec((s.num_heads * self.q_head, s.q_rank), [Source(s.uq_name)]),
            "wuk": ParamSpec((s.num_heads * s.nope_dim, s.kv_rank), [Source(s.uk_name)]),
            "wuv": ParamSpec((s.num_heads * s.v_dim, s.kv_rank), [Source(s.uv_name)]),
            "wo": ParamSpec((s.hidden, s.num_heads * s.v_dim), [Source(s.o_name)]),
        }

    def streamed_params(self) -> list[str]:
        return ["w_in", "wuq", "wo"]

    def scratch_elements_per_token(self) -> int:
        s: LatentAttentionSpec = self.spec
        h = s.num_heads
        return (self.in_rows + s.q_rank + h * self.q_head + 2 * h * s.kv_rank + 2 * h * s.v_dim + s.hidden)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedLatentHandle) -> torch.Tensor:
        s: LatentAttentionSpec = self.spec
        n, h, r = ctx.num_tokens, s.num_heads, s.kv_rank
        proj = ctx.scratch("lat_in", (n, self.in_rows), ctx.dtype)
        linear(x, self.w_in, None, proj, ctx.scratch)
        table, pairing = None, "half"
        if self.position is not None and self.rot_dims:
            table, _ = self.position.rotary(ctx.device)
            pairing = self.position.pairing
        cq = ctx.scratch("lat_cq", (n, s.q_rank), ctx.dtype)
        K.latent_prep(proj, s.q_rank, r, s.rope_dim, self.q_gain, self.kv_gain, s.eps, ctx.positions,
                      ctx.row_of_token, table, self.rot_dims, pairing, cache.pages, cache.block_tables, cq,
                      write=cache.write)
        q = ctx.scratch("lat_q", (n, h * self.q_head), ctx.dtype)
        linear(cq, self.wuq, None, q, ctx.scratch)
        if self.rot_dims:
            K.rope_inplace(q, h, self.q_head, s.nope_dim, self.rot_dims, pairing, ctx.positions, table)
        # the key up-projection folded into the query: qlat[h] = q_plain[h] Wuk[h]
        qlat = ctx.scratch("lat_qlat", (h, n, r), ctx.dtype)
        torch.bmm(q.view(n, h, self.q_head)[:, :, :s.nope_dim].transpose(0, 1),
                  self.wuk.view(h, s.nope_dim, r), out=qlat)
        olat = ctx.scratch("lat_olat", (h, n, r), ctx.dtype)
        # (a block of the tensor-core kernel serves 16 heads, one of the generic kernel 8)
        chunks = -(-h // (16 if ctx.dtype == torch.bfloat16 else 8))
        splits = latent_splits(n, chunks, ctx.max_ctx_len, K.sm_count(ctx.device))
        scratch = None
        if splits > 1:
            nbytes = K.latent_attention_scratch_bytes(n, h, r, splits)
            scratch = ctx.scratch("attn_partials", (nbytes // 4,), torch.float32)
        K.latent_attention(qlat, q, s.nope_dim, self.q_head, cache.pages, cache.block_tables, ctx.positions,
                           ctx.row_of_token, olat, h, r, s.rope_dim, s.scale, splits=splits, scratch=scratch)
        # values of the attended latent: ov[h] = olat[h] Wuv[h]^T
        ov = ctx.scratch("lat_ov", (h, n, s.v_dim), ctx.dtype)
        torch.bmm(olat, self.wuv.view(h, s.v_dim, r).transpose(1, 2), out=ov)
        heads = ctx.scratch("attn_out", (n, h * s.v_dim), ctx.dtype)
        gate = proj[:, self.in_rows - h * s.v_dim:] if s.gated else None
        K.heads_gate(ov, gate, heads)
        y = ctx.scratch("mixer_out", (n, s.hidden), ctx.dtype)
        return linear(heads, self.wo, None, y, ctx.scratch)
