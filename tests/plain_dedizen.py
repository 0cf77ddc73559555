"""A plain, slow implementation of the Dedizen decoder: one function per mechanism, whole
sequences at once, token-by-token recurrences, dense masks, no cache and no batching.  It
shares no code with the package; the tests compare the engine with it.

Notation: a sequence is ``x[t, :]`` with positions t = 0, 1, ...; weights are ``[out, in]``
and act as ``x @ W.T``.  Everything is computed in the dtype the tensors are given in
(the tests use float64).
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ---- reading a model folder ------------------------------------------------------------

def read_safetensors(path) -> dict[str, torch.Tensor]:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = np.frombuffer(data[lo:hi], dtype=np.uint8)
        kind = info["dtype"]
        if kind == "BF16":
            u = buf.view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif kind == "F32":
            t = torch.from_numpy(buf.view(np.float32).copy())
        elif kind == "I32":
            t = torch.from_numpy(buf.view(np.int32).copy())
        else:
            raise ValueError(kind)
        out[name] = t.reshape(info["shape"])
    return out


def read_model_dir(model_dir):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    return cfg, read_safetensors(model_dir / "model.safetensors")


# ---- mechanisms ------------------------------------------------------------------------

def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared_mlp(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def yarn_frequencies(dims, base, scaling, dtype):
    """(frequency of every pair [dims/2], the factor on cos and sin)."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = scaling["factor"], scaling["original"]

    def where(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1


def rotate_interleaved(x, freq, mag):
    """x: [T, heads, dim]; pairs (2i, 2i+1) of the first 2 * len(freq) numbers turn by t * freq[i]."""
    t = torch.arange(x.shape[0], dtype=x.dtype)
    a = t[:, None] * freq[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    d = 2 * freq.numel()
    u, v = x[..., 0:d:2], x[..., 1:d:2]
    out = x.clone()
    out[..., 0:d:2] = u * c - v * s
    out[..., 1:d:2] = v * c + u * s
    return out


def chunked_sink_attention(h, w, p, m, eps):
    """Grouped-query attention whose values are the keys as projected; rotary on part of each head,
    unit-RMS q and k, a chunk mask counted from position 0, a sink in the softmax's denominator
    and a sigmoid gate per head."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = k
    rot = m.get("rot")
    if rot and rot.get("dims"):
        freq, mag = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
        q, k = rotate_interleaved(q, freq, mag), rotate_interleaved(k, freq, mag)
    q, k = rms(q, eps), rms(k, eps)
    t = torch.arange(T)
    seen = t[None, :] <= t[:, None]
    size = (m.get("mask") or {}).get("size")
    if size:
        seen = seen & (t[None, :] // size == t[:, None] // size)
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, H]
    out = torch.zeros(T, H, v.shape[-1], dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        e = torch.exp(s - s.max(-1, keepdim=True).values)
        sink = torch.exp(w[p + "sink"][head] - s.max(-1).values)
        wts = e / (e.sum(-1) + sink)[:, None]
        out[:, head] = (wts @ v[:, kv]) * gate[:, head:head + 1]
    return out.reshape(T, -1) @ w[p + "o"].T


def lightning_attention(h, w, p, m, eps):
    """Linear attention with a fixed decay per head: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w[p + "q"].T).view(T, H, D)
    k = silu(h @ w[p + "k"].T).view(T, H, D)
    v = silu(h @ w[p + "v"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    o = rms(out.reshape(T, -1), eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = chunked_sink_attention(h, w, p + "left.", m["left"], eps)
    right = lightning_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


def mlstm(h, w, p, m, eps):
    """The matrix memory with exponential gating and a running maximum that starts at 0."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    ig = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        n = torch.zeros(D, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            new = torch.maximum(fg[t, head] + mx, ig[t, head])
            a, b = torch.exp(fg[t, head] + mx - new), torch.exp(ig[t, head] - new)
            S = a * S + b * torch.outer(k[t, head], v[t, head])
            n = a * n + b * k[t, head]
            mx = new
            den = torch.maximum(torch.abs(n @ q[t, head]), torch.exp(-mx)) + 1e-6
            out[t, head] = (S.T @ q[t, head]) / den
    o = rms(out, eps).reshape(T, -1) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def rglru(h, w, p, m, eps):
    """Two branches: a gelu branch y, and a causal convolution followed by the gated linear
    recurrence S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t; the output is W_o (S * y)."""
    T = h.shape[0]
    C, B, taps = m["width"], m["blocks"], m["conv"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    x = h @ w[p + "x"].T + w[p + "x.b"]
    xp = torch.cat((torch.zeros(taps - 1, C, dtype=h.dtype), x))
    u = w[p + "conv.b"] + sum(w[p + "conv"][:, j] * xp[j:j + T] for j in range(taps))
    ub = u.view(T, B, C // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, C)
    a = torch.exp(-8 * r * torch.nn.functional.softplus(w[p + "lam"]))
    S = torch.zeros(C, dtype=h.dtype)
    out = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ w[p + "o"].T


MIXERS = {"parallel": parallel_mixer, "mlstm": mlstm, "rglru": rglru}


def forward(cfg, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence; with `layers_out` (a list) the stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](rms(x, eps) * w[p + "norm1"], w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + relu_squared_mlp(rms(x, eps) * w[p + "norm2"], w[p + "mlp.up"], w[p + "mlp.down"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["embed"].T
